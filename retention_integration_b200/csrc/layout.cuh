// Internal layout of the symmetric-power expansion for deg = 2 ("pair-aligned
// triangle").  For head dim d (even) row a holds the products x[a]*x[b] for
// b = 2*floor(a/2) .. d-1, rows stored one after another:
//
//     D2 = d*(d+2)/2            (2112 for d = 64; the exact C(d+1,2) is 2080)
//
// Every row starts at an even b and has even length, so two consecutive entries
// always share `a` and form an aligned pair (x[b], x[b+1]) - the expansion is one
// packed 16-bit multiply per two entries with no shuffling.  The d/2 entries with
// b = a-1 (a odd) duplicate (a-1, a); they carry weight 0 on the key side, so the
// states hold zeros there and the query side may leave its products in place.
// Key-side weights: 1 for a == b, 2 for b > a, 0 for b < a.  (The reference's layout,
// retention/_update_state/reference.py:5-29, pads whole 16x16 diagonal blocks
// instead: 2560 at d = 64.)
#pragma once
#include <stdint.h>

namespace pr {

__host__ __device__ constexpr int t2_dim(int d) { return d * (d + 2) / 2; }

// first entry of row a: rows 2p and 2p+1 both have length d - 2p
__host__ __device__ constexpr int t2_row_offset(int d, int a) {
  const int p = a >> 1;
  return 2 * p * (d - p + 1) + ((a & 1) ? (d - 2 * p) : 0);
}

// entry index -> (a, b)
__host__ __device__ inline void t2_decode(int d, int idx, int* a, int* b) {
  int p = 0;
  while (p + 1 <= d / 2 && 2 * (p + 1) * (d - (p + 1) + 1) <= idx) ++p;
  int rem = idx - 2 * p * (d - p + 1);
  const int len = d - 2 * p;
  if (rem < len) {
    *a = 2 * p;
    *b = 2 * p + rem;
  } else {
    *a = 2 * p + 1;
    *b = 2 * p + rem - len;
  }
}

__host__ __device__ inline float t2_key_weight(int a, int b) { return a == b ? 1.f : (b > a ? 2.f : 0.f); }

}  // namespace pr
