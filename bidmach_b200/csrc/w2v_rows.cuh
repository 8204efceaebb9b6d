// Row-level helpers shared by the update kernels and the bench-only row-traffic probe:
// where an update to a word's row goes (the row, or a replica row of a hot id), and
// loads / atomic additions of a lane's share of a row.
#pragma once

#include "w2v_device.cuh"
#include "w2v_internal.h"

namespace w2v {

// Destination of an update to row w of matrix M: the row itself, or for a hot
// id one of its replica rows in the side buffer (picked by the warp's number).
__device__ __forceinline__ float *update_target(float *M, float *shadow, const HotRows &hot, int w,
                                                int dim, unsigned pick) {
  if (w + 1 < hot.limit) {
    // level L holds the 2^L ids with 2^L <= id + 1 < 2^(L+1), each with rmax >> L replicas
    const int level = 31 - __clz(w + 1);
    const int reps = hot.rmax >> level;
    const int row = hot.rmax * level + (w + 1 - (1 << level)) * reps + (int)(pick & (unsigned)(reps - 1));
    return shadow + (int64_t)row * dim;
  }
  return M + (int64_t)w * dim;
}

// Only the last of a lane's NR vectors can fall off the end of a row (NR is
// ceil(nvec / 32)), so one flag per lane replaces a bounds test per access.
template <int NR>
__device__ __forceinline__ bool vec_ok(int q, bool tail) {
  return q < NR - 1 || tail;
}

// prow_load for a lane that already knows whether its last vector exists;
// `base` points at the lane's first vector.
template <int NR>
__device__ __forceinline__ void prow_load_lane(PRow<NR> &r, const ulonglong2 *base, bool tail) {
#pragma unroll
  for (int q = 0; q < NR; q++) {
    ulonglong2 t = make_ulonglong2(0ull, 0ull);
    if (vec_ok<NR>(q, tail)) t = base[32 * q];
    r.v[q][0] = t.x;
    r.v[q][1] = t.y;
  }
}

// dst[...] += r, `dst` pointing at the lane's first vector of the destination row.
template <int NR>
__device__ __forceinline__ void prow_red_lane(float *dst, bool tail, const PRow<NR> &r) {
#pragma unroll
  for (int q = 0; q < NR; q++) {
    if (vec_ok<NR>(q, tail)) {
      float4 v;
      unpack2(r.v[q][0], v.x, v.y);
      unpack2(r.v[q][1], v.z, v.w);
      red_add_v4(dst + 128 * q, v);
    }
  }
}


}  // namespace w2v
