// Layout of the symmetric-power expansion for deg = 2 used by every kernel and by the chunk
// states in HBM: the reference package's own layout (retention/_update_state/reference.py:5-29,
// retention/_query_state/reference.py:11-33).  With B = 16 and head dim d,
//
//     entry  I(y, a, i) = 256*y*(y+1)/2 + 16*a + i   holds  x[a] * x[16*y + i]
//     for  y in [0, d/16),  a in [0, 16*(y+1)),  i in [0, 16);      DR = 2560 at d = 64.
//
// Every group (y, a) is 16 consecutive entries with a fixed first factor x[a] and an aligned run
// of second factors, so it is 8 packed 16-bit multiplies (x_a,x_a)*(x_b,x_{b+1}) and exactly one
// K = 16 step of tcgen05.mma; the expansion and its gradient are short loops over a with the
// register indices of the second factor known at compile time.  Pairs whose indices fall in the
// same 16-block appear twice, (a,b) and (b,a), each with weight 1; pairs from different blocks
// appear once and carry weight 2 on the key side.  The exact count C(d+1,2) = 2080 is what the
// algorithmic FLOPs are quoted with; the padded layout costs 23 % more tensor work but lets the
// CUDA-core side run from the instruction cache instead of streaming unrolled code.
#pragma once
#include <stdint.h>

namespace pr {

__host__ __device__ constexpr int ref_dim(int d) { return 128 * (d / 16) * (d / 16 + 1); }
// first entry of b-block y
__host__ __device__ constexpr int ref_block_base(int y) { return 128 * y * (y + 1); }

// entry index -> (a, b)
__host__ __device__ inline void ref_decode(int idx, int* a, int* b) {
  int y = 0;
  while (ref_block_base(y + 1) <= idx) ++y;
  const int rem = idx - ref_block_base(y);
  *a = rem >> 4;
  *b = 16 * y + (rem & 15);
}
// key-side weight of entry (a, b): 2 when a lies left of b's 16-block
__host__ __device__ inline float ref_key_weight(int a, int b) { return a < (b & ~15) ? 2.f : 1.f; }

}  // namespace pr
