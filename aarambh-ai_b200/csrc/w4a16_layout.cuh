// Kernel-native layout of a W4A16 weight: tile-major blocks.
//
// Rows are grouped into tiles of 16 and K into quantisation groups.  Block
// (tile, g) holds everything the GEMV needs for 16 rows x one group in one
// contiguous run of words, so a CTA streams its tile with a few large bulk
// copies:
//     16 rows x (group/8) code words   (row r at word r * group/8)
//     16 parameter words               (row r at word 16 * group/8 + r)
// Code words use interleaved slots (slot i holds element {0,2,4,6,1,3,5,7}[i]);
// a parameter word is  bf16 scale | (0xC300 | zero) << 16, i.e. the scale and
// the bf16 value -(128 + zero).  Blocks are ordered [tile][g]; rows beyond N in
// the last tile are zero (scale 0), so they contribute nothing.
#pragma once

#include <stddef.h>
#include <stdint.h>

namespace ab2 {

struct W4Layout {
    int N, K, group;
    __host__ __device__ int G() const { return K / group; }
    __host__ __device__ int tiles() const { return (N + 15) >> 4; }
    __host__ __device__ int words_per_row() const { return group >> 3; }
    __host__ __device__ int block_words() const { return 16 * (group >> 3) + 16; }
    __host__ __device__ size_t total_words() const {
        return (size_t)tiles() * G() * block_words();
    }
    __host__ __device__ size_t block_base(int tile, int g) const {
        return ((size_t)tile * G() + g) * block_words();
    }
    // word `word` (0 .. K/8-1) of row n
    __host__ __device__ size_t code_index(int n, int word) const {
        int wpr = words_per_row();
        return block_base(n >> 4, word / wpr) + (size_t)(n & 15) * wpr + word % wpr;
    }
    __host__ __device__ size_t param_index(int n, int g) const {
        return block_base(n >> 4, g) + (size_t)16 * words_per_row() + (n & 15);
    }
};

}  // namespace ab2
