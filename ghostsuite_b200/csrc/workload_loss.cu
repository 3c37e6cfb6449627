// Token cross-entropy of the benchmark language model, forward and backward, as two streaming
// kernels.  Not part of the ghost hot path and without a counterpart in the reference (its models
// take the loss from torch ops): with a 50304-column vocabulary and 40 x 1024 tokens, the usual
// formulation (fp32 copy of the logits, log-softmax, its backward, casts) moves the 4 GB logit
// tensor through HBM about ten times per step; here the forward reads the logits once (online
// max / sum per row) and the backward reads them once more and writes the gradient once.
//
//   forward : lse[r] = log sum_{c < cols_valid} exp(x[r, c]);  loss[r] = lse[r] - x[r, target[r]]
//             (0 when target[r] == ignore_index)
//   backward: dx[r, c] = scale * (exp(x[r, c] - lse[r]) - [c == target[r]])  for c < cols_valid,
//             0 for padded columns and ignored rows; scale is a device scalar (upstream / n_valid)
//   fused   : the forward also writes dx for an upstream gradient of 1 (its second pass over the
//             row hits L2: the CTA has just read those 100 KB); the backward then only rescales in
//             place, and returns at once when the upstream gradient is exactly 1
#include "common.cuh"

namespace gb {

template <typename T> struct LossVec;
template <> struct LossVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&x)[8]) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      x[2 * e] = __uint_as_float(ww[e] << 16);
      x[2 * e + 1] = __uint_as_float(ww[e] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&x)[8]) {
    uint4 w;
    uint32_t* ww = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
      ww[e] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = w;
  }
  static __device__ __forceinline__ float one(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void put(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct LossVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&x)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&x)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  }
  static __device__ __forceinline__ float one(const float* p) { return *p; }
  static __device__ __forceinline__ void put(float* p, float v) { *p = v; }
};

__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  if (mm == -INFINITY) { m = mm; s = 0.f; return; }
  s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
  m = mm;
}

// one CTA per row
template <typename T>
__global__ void __launch_bounds__(256) ce_forward_kernel(const T* __restrict__ logits, long long ld,
                                                         const long long* __restrict__ targets, int cols_valid,
                                                         long long ignore_index, float* __restrict__ lse_out,
                                                         float* __restrict__ loss_out,
                                                         const float* __restrict__ scale_ptr, int cols,
                                                         T* __restrict__ dlogits, long long ld_out) {
  constexpr int N = LossVec<T>::N;
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  const int full = cols_valid / N * N;
  for (int c = threadIdx.x * N; c < full; c += blockDim.x * N) {
    float v[N];
    LossVec<T>::load(x + c, v);
    float vm = v[0];
#pragma unroll
    for (int e = 1; e < N; ++e) vm = fmaxf(vm, v[e]);
    if (vm > m) { s *= __expf(m - vm); m = vm; }
#pragma unroll
    for (int e = 0; e < N; ++e) s += __expf(v[e] - m);
  }
  for (int c = full + threadIdx.x; c < cols_valid; c += blockDim.x) {
    const float v = LossVec<T>::one(x + c);
    if (v > m) { s *= __expf(m - v); m = v; }
    s += __expf(v - m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    lse_merge(m, s, m2, s2);
  }
  __shared__ float sm[8], ss[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sm[warp] = m; ss[warp] = s; }
  __syncthreads();
  __shared__ float s_lse;
  if (threadIdx.x == 0) {
    for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) lse_merge(m, s, sm[w], ss[w]);
    const float lse = m + logf(s);
    lse_out[row] = lse;
    s_lse = lse;
    const long long t = targets[row];
    loss_out[row] = (t == ignore_index || t < 0 || t >= cols_valid) ? 0.f : lse - LossVec<T>::one(x + t);
  }
  if (dlogits == nullptr) return;
  // fused gradient for an upstream gradient of 1: scale = 1 / (number of counted rows)
  __syncthreads();
  const float l = s_lse;
  T* dx = dlogits + row * ld_out;
  const long long t = targets[row];
  const bool live = !(t == ignore_index || t < 0 || t >= cols_valid);
  const float scale = live ? *scale_ptr : 0.f;
  const int fullc = cols / N * N;
  for (int c = threadIdx.x * N; c < fullc; c += blockDim.x * N) {
    float v[N];
    if (live) {
      LossVec<T>::load(x + c, v);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        const int cc = c + e;
        v[e] = cc < cols_valid ? scale * (__expf(v[e] - l) - (cc == t ? 1.f : 0.f)) : 0.f;
      }
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e) v[e] = 0.f;
    }
    LossVec<T>::store(dx + c, v);
  }
  for (int c = fullc + threadIdx.x; c < cols; c += blockDim.x) {
    float gv = 0.f;
    if (live && c < cols_valid) gv = scale * (__expf(LossVec<T>::one(x + c) - l) - (c == t ? 1.f : 0.f));
    LossVec<T>::put(dx + c, gv);
  }
}

// dx *= upstream[0], skipped entirely when the upstream gradient is exactly 1
template <typename T>
__global__ void __launch_bounds__(256) ce_rescale_kernel(T* __restrict__ dx, long long n_vec,
                                                         const float* __restrict__ upstream) {
  constexpr int N = LossVec<T>::N;
  const float u = *upstream;
  if (u == 1.f) return;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v[N];
    LossVec<T>::load(dx + i * N, v);
#pragma unroll
    for (int e = 0; e < N; ++e) v[e] *= u;
    LossVec<T>::store(dx + i * N, v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ce_backward_kernel(const T* __restrict__ logits, long long ld,
                                                          const long long* __restrict__ targets, int cols,
                                                          int cols_valid, long long ignore_index,
                                                          const float* __restrict__ lse,
                                                          const float* __restrict__ scale_ptr,
                                                          T* __restrict__ dlogits, long long ld_out) {
  constexpr int N = LossVec<T>::N;
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  T* dx = dlogits + row * ld_out;
  const long long t = targets[row];
  const bool live = !(t == ignore_index || t < 0 || t >= cols_valid);
  const float scale = live ? *scale_ptr : 0.f;
  const float l = lse[row];
  const int full = cols / N * N;
  for (int c = threadIdx.x * N; c < full; c += blockDim.x * N) {
    float v[N];
    if (live) {
      LossVec<T>::load(x + c, v);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        const int cc = c + e;
        v[e] = cc < cols_valid ? scale * (__expf(v[e] - l) - (cc == t ? 1.f : 0.f)) : 0.f;
      }
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e) v[e] = 0.f;
    }
    LossVec<T>::store(dx + c, v);
  }
  for (int c = full + threadIdx.x; c < cols; c += blockDim.x) {
    float g = 0.f;
    if (live && c < cols_valid) g = scale * (__expf(LossVec<T>::one(x + c) - l) - (c == t ? 1.f : 0.f));
    LossVec<T>::put(dx + c, g);
  }
}

}  // namespace gb

using namespace gb;

static int check_ce_args(const void* logits, int is_f32, long long rows, int cols, int cols_valid, long long ld,
                         const char* who) {
  GB_REQUIRE(logits != nullptr, "%s: null pointer", who);
  GB_REQUIRE(rows > 0 && rows < (1ll << 31) && cols > 0 && cols_valid > 0 && cols_valid <= cols && ld >= cols,
             "%s: bad shape", who);
  const int vec = is_f32 ? 4 : 8;
  GB_REQUIRE((reinterpret_cast<uintptr_t>(logits) & 15u) == 0 && ld % vec == 0,
             "%s: rows must be 16-byte aligned", who);
  return GHOST_OK;
}

extern "C" int ghost_workload_ce_forward(const void* logits, int is_f32, long long rows, int cols, int cols_valid,
                                         long long ld, const long long* targets, long long ignore_index,
                                         float* lse, float* loss_rows, const float* scale, void* dlogits,
                                         void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  int rc = check_ce_args(logits, is_f32, rows, cols, cols_valid, ld, "ghost_workload_ce_forward");
  if (rc != GHOST_OK) return rc;
  GB_REQUIRE(targets && lse && loss_rows, "ghost_workload_ce_forward: null pointer");
  GB_REQUIRE((dlogits == nullptr) || (scale != nullptr && (reinterpret_cast<uintptr_t>(dlogits) & 15u) == 0 &&
                                      cols % (is_f32 ? 4 : 8) == 0),
             "ghost_workload_ce_forward: the fused gradient needs a scale and 16-byte aligned dense rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_f32)
    ce_forward_kernel<float><<<static_cast<unsigned>(rows), 256, 0, st>>>(
        static_cast<const float*>(logits), ld, targets, cols_valid, ignore_index, lse, loss_rows, scale, cols,
        static_cast<float*>(dlogits), cols);
  else
    ce_forward_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, targets, cols_valid, ignore_index, lse, loss_rows, scale,
        cols, static_cast<__nv_bfloat16*>(dlogits), cols);
  count_launch();
  return post_launch("ce_forward_kernel");
}

extern "C" int ghost_workload_ce_backward(const void* logits, int is_f32, long long rows, int cols, int cols_valid,
                                          long long ld, const long long* targets, long long ignore_index,
                                          const float* lse, const float* scale, void* dlogits, long long ld_out,
                                          void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  int rc = check_ce_args(logits, is_f32, rows, cols, cols_valid, ld, "ghost_workload_ce_backward");
  if (rc != GHOST_OK) return rc;
  GB_REQUIRE(targets && lse && scale && dlogits, "ghost_workload_ce_backward: null pointer");
  const int vec = is_f32 ? 4 : 8;
  GB_REQUIRE((reinterpret_cast<uintptr_t>(dlogits) & 15u) == 0 && ld_out >= cols && ld_out % vec == 0,
             "ghost_workload_ce_backward: output rows must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_f32)
    ce_backward_kernel<float><<<static_cast<unsigned>(rows), 256, 0, st>>>(
        static_cast<const float*>(logits), ld, targets, cols, cols_valid, ignore_index, lse, scale,
        static_cast<float*>(dlogits), ld_out);
  else
    ce_backward_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, targets, cols, cols_valid, ignore_index, lse, scale,
        static_cast<__nv_bfloat16*>(dlogits), ld_out);
  count_launch();
  return post_launch("ce_backward_kernel");
}

extern "C" int ghost_workload_ce_rescale(void* dlogits, int is_f32, long long rows, int cols, const float* upstream,
                                         void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(dlogits && upstream && rows > 0 && cols > 0, "ghost_workload_ce_rescale: bad arguments");
  const int vec = is_f32 ? 4 : 8;
  GB_REQUIRE((reinterpret_cast<uintptr_t>(dlogits) & 15u) == 0 && cols % vec == 0,
             "ghost_workload_ce_rescale: rows must be 16-byte aligned");
  const long long n_vec = rows * cols / vec;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = ds->sm_count * 8;
  if (is_f32) ce_rescale_kernel<float><<<blocks, 256, 0, st>>>(static_cast<float*>(dlogits), n_vec, upstream);
  else ce_rescale_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<__nv_bfloat16*>(dlogits), n_vec, upstream);
  count_launch();
  return post_launch("ce_rescale_kernel");
}
