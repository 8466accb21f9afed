// Shared-segment rows ("SSR" image): a host-side codec for very sparse ternary matrices.
//
// The reference names a sparse-segment encoding but ships no definition of it (SSR/README.md is a citation, and the
// only consumer, the swizzled tile read of ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:159-160, is commented out).  This is
// this library's own encoding in the spirit of the common prefix of MergedTCSC_Group (ternaryLLM_CPU/src/TCSC.hpp:99-145),
// where the columns of a group share one run of row ids: here the 8 columns of a group share, per segment of 256 rows
// of W, ONE ascending list of the rows that any of them uses (one byte each, the offset inside the segment) and, per
// listed row, one 16-bit word of two-bit codes (column i of the group in bits 2i..2i+1: 0 = zero, 1 = +1, 2 = -1).
//
//   image   = header | group_offsets: uint32 [groups + 1], byte offsets into the payload | payload
//   payload = for every group, for every segment:  uint16 n | uint16 codes[n] | uint8 rows[n] | one pad byte if n is odd
//
// so a (group, segment) costs 2 + 3n bytes.  With independent entries n = 256 (1 - zeros^8): 0.215 / 0.127 / 0.057 bytes
// per entry of W at 90 / 95 / 98 % zeros.  Only the codec exists (encode, validating decode); no kernel reads the image.
#include <cstdint>
#include <cstring>
#include <vector>

#include "../../include/tllm.h"
#include "util.h"

namespace {

constexpr uint32_t SSR_MAGIC = 0x31525353u;   // "SSR1"
constexpr int SSR_GROUP = 8, SSR_SEGMENT = 256;

struct SsrHeader {
    uint32_t magic;
    int32_t inners, columns, group, segment;
    uint32_t payload_bytes;
};

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// the listed rows and code words of one (group, segment); returns n
int collect(const int8_t* w, int columns, int n0, int gcols, int k0, int klen, uint16_t* codes, uint8_t* rows) {
    int n = 0;
    for (int r = 0; r < klen; ++r) {
        const int8_t* row = w + (size_t)(k0 + r) * columns + n0;
        uint16_t code = 0;
        for (int i = 0; i < gcols; ++i) code |= (uint16_t)((row[i] > 0 ? 1u : (row[i] < 0 ? 2u : 0u)) << (2 * i));
        if (code) codes[n] = code, rows[n] = (uint8_t)r, ++n;
    }
    return n;
}

}  // namespace

extern "C" int tllm_ssr_encode(const int8_t* w, int inners, int columns, uint8_t* image, size_t capacity, size_t* bytes) {
    if (!w || !bytes || inners <= 0 || columns <= 0) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_encode: bad argument");
    const int groups = ceil_div(columns, SSR_GROUP), segments = ceil_div(inners, SSR_SEGMENT);
    const size_t table_bytes = (size_t)(groups + 1) * sizeof(uint32_t);
    std::vector<uint32_t> offsets((size_t)groups + 1);
    std::vector<uint8_t> payload;
    uint16_t codes[SSR_SEGMENT];
    uint8_t rows[SSR_SEGMENT];
    for (int g = 0; g < groups; ++g) {
        offsets[g] = (uint32_t)payload.size();
        const int n0 = g * SSR_GROUP, gcols = columns - n0 < SSR_GROUP ? columns - n0 : SSR_GROUP;
        for (int s = 0; s < segments; ++s) {
            const int k0 = s * SSR_SEGMENT, klen = inners - k0 < SSR_SEGMENT ? inners - k0 : SSR_SEGMENT;
            const int n = collect(w, columns, n0, gcols, k0, klen, codes, rows);
            const size_t at = payload.size();
            payload.resize(at + 2 + 3 * (size_t)n + (n & 1));
            const uint16_t n16 = (uint16_t)n;
            std::memcpy(&payload[at], &n16, 2);
            std::memcpy(&payload[at + 2], codes, 2 * (size_t)n);
            std::memcpy(&payload[at + 2 + 2 * (size_t)n], rows, (size_t)n);
            if (n & 1) payload[at + 2 + 3 * (size_t)n] = 0;
        }
        if (payload.size() > 0xFFFFFFF0u) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_encode: the image would pass 4 GiB");
    }
    offsets[groups] = (uint32_t)payload.size();
    *bytes = sizeof(SsrHeader) + table_bytes + payload.size();
    if (!image) return TLLM_OK;                                  // size query
    if (capacity < *bytes) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_encode: %zu bytes needed, %zu given", *bytes, capacity);
    const SsrHeader h{SSR_MAGIC, inners, columns, SSR_GROUP, SSR_SEGMENT, (uint32_t)payload.size()};
    std::memcpy(image, &h, sizeof h);
    std::memcpy(image + sizeof h, offsets.data(), table_bytes);
    if (!payload.empty()) std::memcpy(image + sizeof h + table_bytes, payload.data(), payload.size());
    return TLLM_OK;
}

extern "C" int tllm_ssr_decode(const uint8_t* image, size_t bytes, int inners, int columns, int8_t* w_out) {
    if (!image || !w_out || inners <= 0 || columns <= 0) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: bad argument");
    SsrHeader h;
    if (bytes < sizeof h) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: shorter than a header");
    std::memcpy(&h, image, sizeof h);
    if (h.magic != SSR_MAGIC || h.group != SSR_GROUP || h.segment != SSR_SEGMENT) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: not an image of this codec");
    if (h.inners != inners || h.columns != columns)
        return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: the image holds %d x %d, asked for %d x %d", h.inners, h.columns, inners, columns);
    const int groups = ceil_div(columns, SSR_GROUP), segments = ceil_div(inners, SSR_SEGMENT);
    const size_t table_bytes = (size_t)(groups + 1) * sizeof(uint32_t);
    if (bytes != sizeof h + table_bytes + (size_t)h.payload_bytes) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: size does not match the header");
    std::vector<uint32_t> offsets((size_t)groups + 1);
    std::memcpy(offsets.data(), image + sizeof h, table_bytes);
    const uint8_t* payload = image + sizeof h + table_bytes;
    if (offsets[0] != 0 || offsets[groups] != h.payload_bytes) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: group offsets do not span the payload");
    std::memset(w_out, 0, (size_t)inners * (size_t)columns);
    for (int g = 0; g < groups; ++g) {
        if (offsets[g + 1] < offsets[g] || offsets[g + 1] > h.payload_bytes) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: group %d: offsets out of order", g);
        size_t at = offsets[g];
        const size_t end = offsets[g + 1];
        const int n0 = g * SSR_GROUP, gcols = columns - n0 < SSR_GROUP ? columns - n0 : SSR_GROUP;
        for (int s = 0; s < segments; ++s) {
            const int k0 = s * SSR_SEGMENT, klen = inners - k0 < SSR_SEGMENT ? inners - k0 : SSR_SEGMENT;
            if (at + 2 > end) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: group %d ends inside segment %d", g, s);
            uint16_t n16;
            std::memcpy(&n16, payload + at, 2);
            const size_t n = n16, need = 2 + 3 * n + (n & 1);
            if ((int)n > klen || at + need > end) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: group %d segment %d: %zu rows do not fit", g, s, n);
            const uint8_t* codes = payload + at + 2;
            const uint8_t* rows = codes + 2 * n;
            int prev = -1;
            for (size_t i = 0; i < n; ++i) {
                uint16_t code;
                std::memcpy(&code, codes + 2 * i, 2);
                const int r = rows[i];
                if (r <= prev || r >= klen) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: group %d segment %d: row ids not ascending inside the segment", g, s);
                prev = r;
                if (code == 0) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: group %d segment %d: a listed row without an entry", g, s);
                int8_t* out = w_out + (size_t)(k0 + r) * columns + n0;
                for (int c = 0; c < SSR_GROUP; ++c) {
                    const unsigned v = (code >> (2 * c)) & 3u;
                    if (v == 3u || (v && c >= gcols)) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: group %d segment %d: bad code word", g, s);
                    if (v) out[c] = v == 1u ? 1 : -1;
                }
            }
            at += need;
        }
        if (at != end) return tllm::fail(TLLM_ERR_ARG, "tllm_ssr_decode: group %d: %zu bytes left over", g, end - at);
    }
    return TLLM_OK;
}
