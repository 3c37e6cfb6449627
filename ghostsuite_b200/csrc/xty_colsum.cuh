// Per-sample column sums of one GEMM operand (the bias terms' input) taken by four extra warps of
// the per-sample GEMM kernels while the tensor core works on the same rows.
//
// The warps read the operand rows straight from global memory -- L2 hits, because the TMA producer
// is fetching the same rows for the tensor core -- instead of re-reading the shared-memory stages:
// an earlier version did that and slowed the GEMM by two thirds, its reads competing with the
// tensor core's own operand fetch.  No barrier is shared with the pipeline warps; the 128 threads
// synchronise among themselves on a named barrier.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace gb {

// Sums rows [t_begin, t_end) of columns [cbase, cbase + 128) of `src` (row pitch ld, 16-byte aligned,
// column count a multiple of 8) and adds them to out[cbase ..] (zeroed by the host: every unit
// that works on a (sample, column block) takes its share of the sample's rows, so the column-sum
// warps of a unit never have more to read than its tensor-core work covers and read the rows the
// TMA producer is fetching at that moment).  ct = 0..127 is the thread's index among the
// column-sum warps; red is 8 * 128 floats of shared memory; up to sixteen 16-byte loads are in
// flight per thread.
__device__ __forceinline__ void xty_colsum_128(const __nv_bfloat16* __restrict__ src, long long t_begin,
                                               long long T, long long ld, int cbase, int total_cols, float* red,
                                               float* __restrict__ out, int ct, int bar_id) {
  const int cv = ct & 15, rl = ct >> 4;     // 16 column vectors x 8 row lanes
  const int c0 = cbase + cv * 8;
  float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < total_cols) {
    const __nv_bfloat16* base = src + c0;
    auto add8 = [&](const uint4& w) {
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        a[2 * e] += __uint_as_float(ww[e] << 16);
        a[2 * e + 1] += __uint_as_float(ww[e] & 0xffff0000u);
      }
    };
    long long t = t_begin + rl;
    for (; t + 120 < T; t += 128) {
      uint4 w[16];
#pragma unroll
      for (int q = 0; q < 16; ++q) w[q] = __ldg(reinterpret_cast<const uint4*>(base + (t + 8 * q) * ld));
#pragma unroll
      for (int q = 0; q < 16; ++q) add8(w[q]);
    }
    for (; t + 24 < T; t += 32) {
      const uint4 w0 = __ldg(reinterpret_cast<const uint4*>(base + t * ld));
      const uint4 w1 = __ldg(reinterpret_cast<const uint4*>(base + (t + 8) * ld));
      const uint4 w2 = __ldg(reinterpret_cast<const uint4*>(base + (t + 16) * ld));
      const uint4 w3 = __ldg(reinterpret_cast<const uint4*>(base + (t + 24) * ld));
      add8(w0); add8(w1); add8(w2); add8(w3);
    }
    for (; t < T; t += 8) add8(__ldg(reinterpret_cast<const uint4*>(base + t * ld)));
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[rl * 128 + cv * 8 + j] = a[j];
  asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
  float sum = 0.f;
#pragma unroll
  for (int r = 0; r < 8; ++r) sum += red[r * 128 + ct];
  if (cbase + ct < total_cols && sum != 0.f) atomicAdd(out + cbase + ct, sum);
  asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
}

}  // namespace gb
