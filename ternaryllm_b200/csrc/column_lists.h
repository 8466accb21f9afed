// column_lists.h -- column-major view of a row-major ternary matrix, shared by the host packers.
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

namespace tllm {

// Column-major view of a row-major ternary matrix: for every column the ascending row ids of the +1 and
// of the -1 entries.  Built with a counting pass and a scatter pass so that the matrix is read row by row.
template <typename WT>
struct ColumnLists {
    std::vector<int64_t> pos_ptr, neg_ptr;   // columns+1
    std::vector<int32_t> pos_row, neg_row;
    ColumnLists(const WT* w, int inners, int columns) : pos_ptr(columns + 1, 0), neg_ptr(columns + 1, 0) {
        for (int k = 0; k < inners; ++k) {
            const WT* row = w + (size_t)k * columns;
            for (int n = 0; n < columns; ++n) {
                pos_ptr[n + 1] += row[n] > 0;
                neg_ptr[n + 1] += row[n] < 0;
            }
        }
        for (int n = 0; n < columns; ++n) {
            pos_ptr[n + 1] += pos_ptr[n];
            neg_ptr[n + 1] += neg_ptr[n];
        }
        pos_row.resize(pos_ptr[columns]);
        neg_row.resize(neg_ptr[columns]);
        std::vector<int64_t> pc(pos_ptr.begin(), pos_ptr.end() - 1), nc(neg_ptr.begin(), neg_ptr.end() - 1);
        for (int k = 0; k < inners; ++k) {
            const WT* row = w + (size_t)k * columns;
            for (int n = 0; n < columns; ++n) {
                if (row[n] > 0) pos_row[pc[n]++] = k;
                else if (row[n] < 0) neg_row[nc[n]++] = k;
            }
        }
    }
};

}  // namespace tllm
