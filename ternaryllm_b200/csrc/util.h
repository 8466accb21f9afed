// util.h -- error reporting shared by the host sources of libtllm.
#pragma once
#include <cstdint>
#include <vector>

namespace tllm {

// Records a printf-style message for the calling thread (returned by tllm_last_error) and returns `code`.
int fail(int code, const char* fmt, ...);

// counts one kernel launch (tllm_launch_count)
void note_launch();

// decoders of the reference's formats into dense int8 [inners][columns]; return nullptr or a message
const char* decode_mcsc(const int32_t* row_idx, const int32_t* off, int columns, int inners, int tile_k,
                        std::vector<int8_t>* out);
const char* decode_cpu_format(int kind, int group, int chunk, const int32_t* meta, const void* ri, int ri32,
                              int64_t aux, int columns, int inners, std::vector<int8_t>* out);

}  // namespace tllm
