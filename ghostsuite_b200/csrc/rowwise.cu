// Bandwidth-bound kernels of the ghost hot path: dtype cast / bf16 split, per-sample column sums
// (bias terms), per-sample LayerNorm gradients, tiny [n_val x n_train] Grams of per-sample vectors,
// and row sums that turn per-sample vectors into averaged train gradients.  All of them stream
// their inputs once with 16-byte coalesced loads and reduce with warp shuffles / shared memory.
#include "common.cuh"

namespace gb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// 8 consecutive elements -> fp32
template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&x)[8]) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      x[2 * e] = __uint_as_float(ww[e] << 16);
      x[2 * e + 1] = __uint_as_float(ww[e] & 0xffff0000u);
    }
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&x)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
};
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// ------------------------------------------------------------------------------------------
// cast / split.  dst is bf16 with `parts` copies of the (zero-padded) source laid out either
// side by side along columns (col_stack) or one below the other inside each sample (row_stack).
// part kinds: 0 = bf16(x) ("hi"), 1 = bf16(x - hi) ("lo").
// ------------------------------------------------------------------------------------------
struct CastParams {
  const void* src;
  __nv_bfloat16* dst;
  long long samples, T;     // rows = samples * T
  int cols, cpad;           // cpad = padded column count of one part
  long long ld_src, ld_dst;
  int parts;
  int kind[3];
  int row_stack;            // 0: parts side by side; 1: parts stacked along rows within a sample
};

template <typename T>
__global__ void cast_split_kernel(const CastParams p) {
  const long long rows = p.samples * p.T;
  const int cvec = p.cpad / 8;
  const long long total = rows * cvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / cvec;
    const int c0 = static_cast<int>(i % cvec) * 8;
    float x[8];
    const T* src = static_cast<const T*>(p.src) + row * p.ld_src + c0;
    if (c0 + 8 <= p.cols && (reinterpret_cast<uintptr_t>(src) & (sizeof(T) == 4 ? 15u : 15u)) == 0) {
      Vec8<T>::load(src, x);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = (c0 + j < p.cols) ? to_f32<T>(src[j]) : 0.f;
    }
    const long long s = row / p.T, t = row % p.T;
#pragma unroll
    for (int part = 0; part < 3; ++part) {
      if (part >= p.parts) break;
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float a = x[2 * e], b = x[2 * e + 1];
        __nv_bfloat16 ha = __float2bfloat16_rn(a), hb = __float2bfloat16_rn(b);
        if (p.kind[part] == 1) {
          ha = __float2bfloat16_rn(a - __bfloat162float(ha));
          hb = __float2bfloat16_rn(b - __bfloat162float(hb));
        }
        w[e] = static_cast<uint32_t>(__bfloat16_as_ushort(ha)) |
               (static_cast<uint32_t>(__bfloat16_as_ushort(hb)) << 16);
      }
      long long off;
      if (p.row_stack) off = ((s * p.parts + part) * p.T + t) * p.ld_dst + c0;
      else off = row * p.ld_dst + static_cast<long long>(part) * p.cpad + c0;
      *reinterpret_cast<uint4*>(p.dst + off) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------
// per-sample column sums: out[n, c] += sum_{t in split} G[n, t, c]
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void colsum_kernel(const T* __restrict__ G, long long Tn, int cols, long long ld,
                              float* __restrict__ out, int t_splits) {
  // block: 32 column vectors (256 columns) x 8 row lanes
  __shared__ float red[8][256 + 8];
  const int n = blockIdx.z;
  const int split = blockIdx.y;
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c0 = (blockIdx.x * 32 + cx) * 8;
  const long long per = (Tn + t_splits - 1) / t_splits;
  const long long t0 = split * per;
  const long long t1 = (t0 + per < Tn) ? t0 + per : Tn;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const bool vec_ok = (c0 + 8 <= cols) && (ld % 8 == 0) &&
                      ((reinterpret_cast<uintptr_t>(G + static_cast<long long>(n) * Tn * ld + c0) & 15u) == 0);
  if (c0 < cols) {
    const T* base = G + static_cast<long long>(n) * Tn * ld + c0;
    long long t = t0 + ry;
    if (vec_ok) {
      // four independent 16-byte loads in flight per thread
      for (; t + 24 < t1; t += 32) {
        float x0[8], x1[8], x2[8], x3[8];
        Vec8<T>::load(base + t * ld, x0);
        Vec8<T>::load(base + (t + 8) * ld, x1);
        Vec8<T>::load(base + (t + 16) * ld, x2);
        Vec8<T>::load(base + (t + 24) * ld, x3);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += (x0[j] + x1[j]) + (x2[j] + x3[j]);
      }
    }
    for (; t < t1; t += 8) {
      float x[8];
      if (vec_ok) {
        Vec8<T>::load(base + t * ld, x);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = (c0 + j < cols) ? to_f32<T>(base[t * ld + j]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += x[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[ry][cx * 8 + j] = acc[j];
  __syncthreads();
  const int c = threadIdx.x;   // 256 threads, one column each
  float s = 0.f;
#pragma unroll
  for (int r = 0; r < 8; ++r) s += red[r][c];
  const int col = blockIdx.x * 256 + c;
  if (col < cols) {
    float* dst = out + static_cast<long long>(n) * cols + col;
    if (t_splits > 1) atomicAdd(dst, s); else *dst = s;
  }
}

// ------------------------------------------------------------------------------------------
// LayerNorm per-sample gradients, one warp per token row, F <= 256 * NCHUNK, F % 8 == 0.
//   gw[n, f] += sum_t G[n,t,f] * xhat[n,t,f],   gb[n, f] += sum_t G[n,t,f]
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Each warp streams its token rows through a private three-slot ring in shared memory filled with
// cp.async: the loads of the next two rows are in flight while the current row goes through its two
// dependent shuffle reductions.  A lane reads back exactly the 16-byte pieces it copied itself, so
// the ring needs no synchronisation beyond cp.async.wait_group.
constexpr int kLnSlots = 3;

template <typename T, int NCHUNK>
__global__ void __launch_bounds__(256, NCHUNK <= 3 ? 2 : 1)
layernorm_persample_kernel(const T* __restrict__ A, const T* __restrict__ G, long long Tn, int F,
                           float eps, float* __restrict__ gw, float* __restrict__ gb,
                           float* __restrict__ part, int t_splits, int rms) {
  extern __shared__ __align__(16) unsigned char sm_raw[];   // rings [8 warps][3][2][F] of T, then [8][2][F] floats
  float* sm = reinterpret_cast<float*>(sm_raw);
  const int n = blockIdx.y, split = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* ring = reinterpret_cast<T*>(sm_raw) + static_cast<size_t>(warp) * kLnSlots * 2 * F;
  const long long per = (Tn + t_splits - 1) / t_splits;
  const long long t0 = split * per;
  const long long t1 = (t0 + per < Tn) ? t0 + per : Tn;
  float aw[NCHUNK][8], ab[NCHUNK][8];
#pragma unroll
  for (int i = 0; i < NCHUNK; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { aw[i][j] = 0.f; ab[i][j] = 0.f; }
  const float invF = 1.f / static_cast<float>(F);

  auto issue = [&](long long t, int slot) {
    if (t < t1) {
      const long long off = (static_cast<long long>(n) * Tn + t) * F;
      T* sa = ring + static_cast<size_t>(slot) * 2 * F;
      T* sg = sa + F;
#pragma unroll
      for (int i = 0; i < NCHUNK; ++i) {
        const int f = (i * 32 + lane) * 8;
        if (f < F) {
#pragma unroll
          for (int b = 0; b < static_cast<int>(8 * sizeof(T)); b += 16) {
            cp_async16(reinterpret_cast<unsigned char*>(sa + f) + b, reinterpret_cast<const unsigned char*>(A + off + f) + b);
            cp_async16(reinterpret_cast<unsigned char*>(sg + f) + b, reinterpret_cast<const unsigned char*>(G + off + f) + b);
          }
        }
      }
    }
    cp_async_commit();      // an empty group keeps the group count uniform at the tail
  };

  long long t = t0 + warp;
  issue(t, 0);
  issue(t + 8, 1);
  int slot = 0;
  for (; t < t1; t += 8) {
    issue(t + 16, slot == 0 ? 2 : slot - 1);
    cp_async_wait<kLnSlots - 1>();
    const T* sa = ring + static_cast<size_t>(slot) * 2 * F;
    const T* sg = sa + F;
    slot = (slot + 1 == kLnSlots) ? 0 : slot + 1;
    float x[NCHUNK][8], g[NCHUNK][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
      const int f = (i * 32 + lane) * 8;
      if (f < F) {
        Vec8<T>::load(sa + f, x[i]);
        Vec8<T>::load(sg + f, g[i]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) { x[i][j] = 0.f; g[i][j] = 0.f; }
      }
    }
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) s += x[i][j];
    const float mean = rms ? 0.f : warp_sum(s) * invF;     // RMS norm: no centring
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
      const int f = (i * 32 + lane) * 8;
      if (f < F) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { x[i][j] -= mean; q += x[i][j] * x[i][j]; }
      }
    }
    const float rstd = rsqrtf(warp_sum(q) * invF + eps);
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        aw[i][j] = fmaf(g[i][j], x[i][j] * rstd, aw[i][j]);
        ab[i][j] += g[i][j];
      }
  }
  cp_async_wait<0>();
  __syncthreads();          // the rings are reused as the cross-warp reduction scratch
  float* mine = sm + static_cast<size_t>(warp) * 2 * F;
#pragma unroll
  for (int i = 0; i < NCHUNK; ++i) {
    const int f = (i * 32 + lane) * 8;
    if (f < F) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { mine[f + j] = aw[i][j]; mine[F + f + j] = ab[i][j]; }
    }
  }
  __syncthreads();
  for (int f = threadIdx.x; f < 2 * F; f += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) v += sm[static_cast<size_t>(w) * 2 * F + f];
    if (t_splits > 1) {
      part[(static_cast<long long>(split) * gridDim.y + n) * 2 * F + f] = v;
    } else if (f < F) {
      gw[static_cast<long long>(n) * F + f] = v;
    } else {
      gb[static_cast<long long>(n) * F + f - F] = v;
    }
  }
}

// second stage: sum the per-split partials in a fixed order (deterministic)
__global__ void layernorm_reduce_kernel(const float* __restrict__ part, int N, int F, int t_splits,
                                        float* __restrict__ gw, float* __restrict__ gb) {
  const long long total = static_cast<long long>(N) * 2 * F;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < t_splits; ++s) v += part[static_cast<long long>(s) * total + i];
    const int n = static_cast<int>(i / (2 * F)), f = static_cast<int>(i % (2 * F));
    if (f < F) gw[static_cast<long long>(n) * F + f] = v;
    else gb[static_cast<long long>(n) * F + f - F] = v;
  }
}

// generic F: one block per (sample, split); rows handled one at a time by the whole block
template <typename T>
__global__ void __launch_bounds__(256)
layernorm_persample_generic_kernel(const T* __restrict__ A, const T* __restrict__ G, long long Tn, int F,
                                   float eps, float* __restrict__ gw, float* __restrict__ gb, int t_splits,
                                   int rms) {
  extern __shared__ float sm[];   // [2][F] + 32
  float* s_gw = sm;
  float* s_gb = sm + F;
  float* s_red = sm + 2 * F;
  const int n = blockIdx.y, split = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 2 * F; i += blockDim.x) sm[i] = 0.f;
  const long long per = (Tn + t_splits - 1) / t_splits;
  const long long t0 = split * per;
  const long long t1 = (t0 + per < Tn) ? t0 + per : Tn;
  const float invF = 1.f / static_cast<float>(F);
  for (long long t = t0; t < t1; ++t) {
    const T* a = A + (static_cast<long long>(n) * Tn + t) * F;
    const T* g = G + (static_cast<long long>(n) * Tn + t) * F;
    float s = 0.f;
    for (int f = threadIdx.x; f < F; f += blockDim.x) s += to_f32<T>(a[f]);
    s = warp_sum(s);
    __syncthreads();
    if (lane == 0) s_red[warp] = s;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += s_red[w];
    const float mean = rms ? 0.f : tot * invF;
    float q = 0.f;
    for (int f = threadIdx.x; f < F; f += blockDim.x) { const float dlt = to_f32<T>(a[f]) - mean; q += dlt * dlt; }
    q = warp_sum(q);
    __syncthreads();
    if (lane == 0) s_red[warp] = q;
    __syncthreads();
    tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += s_red[w];
    const float rstd = rsqrtf(tot * invF + eps);
    for (int f = threadIdx.x; f < F; f += blockDim.x) {
      const float gv = to_f32<T>(g[f]);
      s_gw[f] += gv * (to_f32<T>(a[f]) - mean) * rstd;   // each f is owned by one thread
      s_gb[f] += gv;
    }
  }
  __syncthreads();
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    const long long o = static_cast<long long>(n) * F + f;
    if (t_splits > 1) { atomicAdd(&gw[o], s_gw[f]); atomicAdd(&gb[o], s_gb[f]); }
    else { gw[o] = s_gw[f]; gb[o] = s_gb[f]; }
  }
}

// ------------------------------------------------------------------------------------------
// M[v, b] = scale * <X[n_train + v, :], X[b, :]>   (one warp per pair)
// ------------------------------------------------------------------------------------------
__global__ void small_gram_kernel(const float* __restrict__ X, int n_train, int n_val, int F,
                                  float scale, float* __restrict__ M) {
  const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (pair >= n_train * n_val) return;
  const int v = pair / n_train, b = pair % n_train;
  const float* xv = X + static_cast<long long>(n_train + v) * F;
  const float* xb = X + static_cast<long long>(b) * F;
  float s = 0.f;
  if ((F & 3) == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0) {
    // 16-byte loads, eight of them in flight per lane before the first use
    const float4* xv4 = reinterpret_cast<const float4*>(xv);
    const float4* xb4 = reinterpret_cast<const float4*>(xb);
    const int F4 = F >> 2;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 4
    for (int f = lane; f < F4; f += 32) {
      const float4 a = __ldg(xv4 + f), c = __ldg(xb4 + f);
      s = fmaf(a.x, c.x, s); s1 = fmaf(a.y, c.y, s1); s2 = fmaf(a.z, c.z, s2); s3 = fmaf(a.w, c.w, s3);
    }
    s = (s + s1) + (s2 + s3);
  } else {
    for (int f = lane; f < F; f += 32) s = fmaf(xv[f], xb[f], s);
  }
  s = warp_sum(s);
  if (lane == 0) M[pair] = s * scale;
}

// out[c] = (accumulate ? out[c] : 0) + scale * sum_{n < n_rows} X[n, c]
template <typename OutT>
__global__ void rows_sum_kernel(const float* __restrict__ X, int n_rows, int F, float scale,
                                OutT* __restrict__ out, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= F) return;
  float s = 0.f;
#pragma unroll 8
  for (int n = 0; n < n_rows; ++n) s += __ldg(X + static_cast<long long>(n) * F + c);
  s *= scale;
  if (accumulate) s += static_cast<float>(out[c]);
  out[c] = static_cast<OutT>(s);
}

// Many small reductions in one launch: job j (blockIdx.y) is the pair of reductions the bias /
// LayerNorm / RMS-norm terms of one layer need on its per-sample vectors X[n_train + n_val, F]:
//   M[v, b]  = dot_scale * <X[n_train + v], X[b]>          (if M != null)
//   sum[c]   = sum_scale * sum_{b < n_train} X[b, c]       (if sum_out != null)
// A backward pass of a GPT-2-sized model has about a hundred of these, each a few microseconds of
// work; the jobs travel as kernel parameters (by value), so the launch is self-contained.
static constexpr int kSmallJobsPerLaunch = 48;
struct SmallJobs {
  ghost_small_job job[kSmallJobsPerLaunch];
};

__global__ void __launch_bounds__(256) small_reduce_batch_kernel(const __grid_constant__ SmallJobs jobs) {
  const ghost_small_job& j = jobs.job[blockIdx.y];
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * 8;
  const float* X = j.X;
  const int F = j.F;
  if (j.M != nullptr) {
    const int pairs = j.n_train * j.n_val;
    const bool vec = (F & 3) == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0;
    for (int pair = blockIdx.x * 8 + (threadIdx.x >> 5); pair < pairs; pair += warps) {
      const int v = pair / j.n_train, b = pair % j.n_train;
      const float* xv = j.Xv == nullptr
                            ? X + static_cast<long long>(j.n_train + v) * F
                            : j.Xv + static_cast<long long>(v / j.v_per_rank) * j.v_rank_pitch +
                                  static_cast<long long>(v % j.v_per_rank) * F;
      const float* xb = X + static_cast<long long>(b) * F;
      float s = 0.f;
      if (vec && (reinterpret_cast<uintptr_t>(xv) & 15) == 0) {
        const float4* xv4 = reinterpret_cast<const float4*>(xv);
        const float4* xb4 = reinterpret_cast<const float4*>(xb);
        const int F4 = F >> 2;
        float s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 4
        for (int f = lane; f < F4; f += 32) {
          const float4 a = __ldg(xv4 + f), c = __ldg(xb4 + f);
          s = fmaf(a.x, c.x, s); s1 = fmaf(a.y, c.y, s1); s2 = fmaf(a.z, c.z, s2); s3 = fmaf(a.w, c.w, s3);
        }
        s = (s + s1) + (s2 + s3);
      } else {
        for (int f = lane; f < F; f += 32) s = fmaf(xv[f], xb[f], s);
      }
      s = warp_sum(s);
      if (lane == 0) j.M[pair] = s * j.dot_scale;
    }
  }
  if (j.sum_out != nullptr) {
    for (int c = blockIdx.x * 256 + threadIdx.x; c < F; c += gridDim.x * 256) {
      float s = 0.f;
#pragma unroll 8
      for (int n = 0; n < j.n_train; ++n) s += __ldg(X + static_cast<long long>(n) * F + c);
      s *= j.sum_scale;
      if (j.sum_is_f32) static_cast<float*>(j.sum_out)[c] = s;
      else static_cast<__nv_bfloat16*>(j.sum_out)[c] = __float2bfloat16_rn(s);
    }
  }
}

}  // namespace gb

using namespace gb;

extern "C" int ghost_small_reduce_batch(const ghost_small_job* jobs, int n_jobs, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(jobs != nullptr && n_jobs > 0, "ghost_small_reduce_batch: no jobs");
  for (int i = 0; i < n_jobs; ++i) {
    const ghost_small_job& j = jobs[i];
    GB_REQUIRE(j.X != nullptr && (j.M != nullptr || j.sum_out != nullptr), "ghost_small_reduce_batch: job %d has no input or no output", i);
    GB_REQUIRE(j.n_train > 0 && j.F > 0 && j.n_val >= 0 && (j.M == nullptr || j.n_val > 0),
               "ghost_small_reduce_batch: job %d has an empty dimension", i);
    GB_REQUIRE(j.Xv == nullptr || (j.v_per_rank > 0 && j.v_rank_pitch >= static_cast<long long>(j.v_per_rank) * j.F),
               "ghost_small_reduce_batch: job %d has separate validation rows without a valid layout", i);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int first = 0; first < n_jobs; first += kSmallJobsPerLaunch) {
    const int n = (n_jobs - first < kSmallJobsPerLaunch) ? n_jobs - first : kSmallJobsPerLaunch;
    SmallJobs batch = {};
    for (int i = 0; i < n; ++i) batch.job[i] = jobs[first + i];
    small_reduce_batch_kernel<<<dim3(8, n, 1), 256, 0, st>>>(batch);
    count_launch();
    const int rc = post_launch("small_reduce_batch_kernel");
    if (rc != GHOST_OK) return rc;
  }
  return GHOST_OK;
}

extern "C" int ghost_cast_split_bf16(const void* src, int src_is_f32, long long samples, long long T,
                                     int cols, long long ld_src, void* dst, long long ld_dst, int cpad,
                                     int parts, int kind0, int kind1, int kind2, int row_stack,
                                     void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(src && dst, "ghost_cast_split_bf16: null pointer");
  GB_REQUIRE(samples > 0 && T > 0 && cols > 0, "ghost_cast_split_bf16: empty input");
  GB_REQUIRE(parts >= 1 && parts <= 3, "ghost_cast_split_bf16: parts must be 1..3");
  GB_REQUIRE(cpad % 8 == 0 && cpad >= cols, "ghost_cast_split_bf16: cpad must be a multiple of 8 and >= cols");
  GB_REQUIRE(ld_dst % 8 == 0 && ld_dst >= (row_stack ? cpad : parts * cpad), "ghost_cast_split_bf16: bad destination pitch");
  GB_REQUIRE((reinterpret_cast<uintptr_t>(dst) & 15u) == 0,
             "ghost_cast_split_bf16: destination must be 16-byte aligned");
  CastParams p;
  p.src = src;
  p.dst = static_cast<__nv_bfloat16*>(dst);
  p.samples = samples;
  p.T = T;
  p.cols = cols;
  p.cpad = cpad;
  p.ld_src = ld_src;
  p.ld_dst = ld_dst;
  p.parts = parts;
  p.kind[0] = kind0; p.kind[1] = kind1; p.kind[2] = kind2;
  p.row_stack = row_stack;
  const long long total = samples * T * (cpad / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > ds->sm_count * 16) blocks = ds->sm_count * 16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (src_is_f32) cast_split_kernel<float><<<static_cast<int>(blocks), 256, 0, st>>>(p);
  else cast_split_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(p);
  count_launch();
  return post_launch("cast_split_kernel");
}

static int pick_splits(long long Tn, long long ctas_without_split, int sm_count, int rows_per_cta_min) {
  long long want = (4ll * sm_count + ctas_without_split - 1) / ctas_without_split;
  long long maxs = (Tn + rows_per_cta_min - 1) / rows_per_cta_min;
  if (want > maxs) want = maxs;
  if (want < 1) want = 1;
  if (want > 65535) want = 65535;
  return static_cast<int>(want);
}

extern "C" int ghost_colsum(const void* G, int is_f32, int N, long long T, int cols, long long ld,
                            float* out, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(G && out, "ghost_colsum: null pointer");
  GB_REQUIRE(N > 0 && T > 0 && cols > 0 && N <= 65535, "ghost_colsum: bad dimensions");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int cblocks = ceil_div(cols, 256);
  const int splits = pick_splits(T, static_cast<long long>(cblocks) * N, ds->sm_count, 64);
  if (splits > 1) GB_CUDA_OK(cudaMemsetAsync(out, 0, sizeof(float) * static_cast<size_t>(N) * cols, st));
  dim3 grid(cblocks, splits, N);
  if (is_f32) colsum_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(G), T, cols, ld, out, splits);
  else colsum_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(G), T, cols, ld, out, splits);
  count_launch();
  return post_launch("colsum_kernel");
}

static int ln_splits(long long Tn, int N, int sm_count) {
  long long want = (2ll * sm_count) / N;   // at most two resident CTAs per SM: one wave
  const long long maxs = (Tn + 63) / 64;
  if (want > maxs) want = maxs;
  if (want < 1) want = 1;
  if (want > 65535) want = 65535;
  return static_cast<int>(want);
}

extern "C" long long ghost_layernorm_workspace_bytes(int N, long long T, int F) {
  // upper bound over devices: at most 1024 splits are ever used
  long long splits = (T + 63) / 64;
  if (splits > 1024) splits = 1024;
  return splits * N * 2 * F * 4 + 256;
}

template <typename T>
static int launch_ln(const T* A, const T* G, int N, long long Tn, int F, float eps, float* gw, float* gb,
                     float* ws, long long ws_bytes, const DeviceState* ds, cudaStream_t st, int rms) {
  const bool fast = (F % 8 == 0) && (F <= 1024) &&
                    ((reinterpret_cast<uintptr_t>(A) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(G) & 15u) == 0);
  if (fast) {
    int splits = ln_splits(Tn, N, ds->sm_count);
    if (splits > 1024) splits = 1024;
    if (splits > 1) {
      GB_REQUIRE(ws && ws_bytes >= static_cast<long long>(splits) * N * 2 * F * 4,
                 "ghost_layernorm_persample: workspace too small");
    }
    dim3 grid(splits, N);
    // per-warp cp.async rings (3 slots x (A row + G row)), reused for the cross-warp reduction
    const size_t ring = sizeof(T) * 8 * kLnSlots * 2 * static_cast<size_t>(F);
    const size_t red = sizeof(float) * 8 * 2 * static_cast<size_t>(F);
    const size_t smem = ring > red ? ring : red;
    const int nchunk = (F + 255) / 256;
#define GB_LN_LAUNCH(NC)                                                                              \
    do {                                                                                              \
      if (smem > 48 * 1024)                                                                           \
        GB_CUDA_OK(cudaFuncSetAttribute(layernorm_persample_kernel<T, NC>,                            \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));    \
      layernorm_persample_kernel<T, NC><<<grid, 256, smem, st>>>(A, G, Tn, F, eps, gw, gb, ws, splits, rms); \
    } while (0)
    switch (nchunk) {
      case 1: GB_LN_LAUNCH(1); break;
      case 2: GB_LN_LAUNCH(2); break;
      case 3: GB_LN_LAUNCH(3); break;
      default: GB_LN_LAUNCH(4); break;
    }
#undef GB_LN_LAUNCH
    count_launch();
    int rc = post_launch("layernorm_persample_kernel");
    if (rc != GHOST_OK || splits == 1) return rc;
    const long long total = static_cast<long long>(N) * 2 * F;
    long long blocks = (total + 255) / 256;
    if (blocks > ds->sm_count * 8) blocks = ds->sm_count * 8;
    layernorm_reduce_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(ws, N, F, splits, gw, gb);
    count_launch();
    return post_launch("layernorm_reduce_kernel");
  }
  const int splits = pick_splits(Tn, N, ds->sm_count, 32);
  if (splits > 1) {
    GB_CUDA_OK(cudaMemsetAsync(gw, 0, sizeof(float) * static_cast<size_t>(N) * F, st));
    GB_CUDA_OK(cudaMemsetAsync(gb, 0, sizeof(float) * static_cast<size_t>(N) * F, st));
  }
  dim3 grid(splits, N);
  const size_t smem = sizeof(float) * (2 * static_cast<size_t>(F) + 32);
  if (smem > 48 * 1024)
    GB_CUDA_OK(cudaFuncSetAttribute(layernorm_persample_generic_kernel<T>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  layernorm_persample_generic_kernel<T><<<grid, 256, smem, st>>>(A, G, Tn, F, eps, gw, gb, splits, rms);
  count_launch();
  return post_launch("layernorm_persample_generic_kernel");
}

static int norm_persample(const char* who, const void* A, const void* G, int is_f32, int N, long long T, int F,
                          float eps, float* gw, float* gb, void* ws, long long ws_bytes, void* stream, int rms) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(A && G && gw && gb, "%s: null pointer", who);
  GB_REQUIRE(N > 0 && T > 0 && F > 0 && N <= 65535, "%s: bad dimensions", who);
  GB_REQUIRE(F <= 24 * 1024, "%s: normalized size above 24576 is not supported", who);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* w = static_cast<float*>(ws);
  if (is_f32) return launch_ln<float>(static_cast<const float*>(A), static_cast<const float*>(G), N, T, F, eps, gw, gb, w, ws_bytes, ds, st, rms);
  return launch_ln<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(G), N, T, F, eps, gw, gb, w, ws_bytes, ds, st, rms);
}

extern "C" int ghost_layernorm_persample(const void* A, const void* G, int is_f32, int N, long long T,
                                         int F, float eps, float* gw, float* gb, void* ws,
                                         long long ws_bytes, void* stream) {
  return norm_persample("ghost_layernorm_persample", A, G, is_f32, N, T, F, eps, gw, gb, ws, ws_bytes, stream, 0);
}

extern "C" int ghost_rmsnorm_persample(const void* A, const void* G, int is_f32, int N, long long T,
                                       int F, float eps, float* gw, float* gsum, void* ws,
                                       long long ws_bytes, void* stream) {
  return norm_persample("ghost_rmsnorm_persample", A, G, is_f32, N, T, F, eps, gw, gsum, ws, ws_bytes, stream, 1);
}

extern "C" int ghost_small_gram_f32(const float* X, int n_train, int n_val, int F, float scale,
                                    float* M_out, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(X && M_out, "ghost_small_gram_f32: null pointer");
  GB_REQUIRE(n_train > 0, "No training samples to compute dot product, check batch sizes.");
  GB_REQUIRE(n_val > 0 && F > 0, "ghost_small_gram_f32: bad dimensions");
  const int pairs = n_train * n_val;
  small_gram_kernel<<<ceil_div(pairs, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(X, n_train, n_val, F, scale, M_out);
  count_launch();
  return post_launch("small_gram_kernel");
}

extern "C" int ghost_rows_sum(const float* X, int n_rows, int F, float scale, void* out, int out_is_f32,
                              int accumulate, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(X && out, "ghost_rows_sum: null pointer");
  GB_REQUIRE(n_rows > 0 && F > 0, "ghost_rows_sum: bad dimensions");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_is_f32) rows_sum_kernel<float><<<ceil_div(F, 64), 64, 0, st>>>(X, n_rows, F, scale, static_cast<float*>(out), accumulate);
  else rows_sum_kernel<__nv_bfloat16><<<ceil_div(F, 64), 64, 0, st>>>(X, n_rows, F, scale, static_cast<__nv_bfloat16*>(out), accumulate);
  count_launch();
  return post_launch("rows_sum_kernel");
}
