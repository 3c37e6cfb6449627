// Embedding-table terms of the ghost hot path (index / gather work, HBM- and latency-bound).
//
// embedding_dot:  M[v, b] = sum_{t, s : id_b[t] == id_v[s]} <G_b[t], G_v[s]>
//   The reference scatters the validation rows into a [vocab, d] table and gathers it at the train
//   ids (ghostEngines/supported_layers_grad_samplers_dotprod.py:203-210); here the validation
//   tokens are chained per token id in a vocab-sized head table (4 bytes per id) and every train
//   token walks the chain of its id, so no [vocab, d] scratch exists and the result is split per
//   validation sample.
//
// embedding_wgrad: averaged train gradient of the table (:214-235).  Train tokens are bucketed by
//   id (count, scan, fill), each bucket is put in ascending token order and summed in float32 in
//   that order, rounded to the table dtype once, then divided by n_train -- the arithmetic and
//   the order of the CPU index_add_, so the result is bit-identical to it.
#include <limits.h>

#include <mutex>

#include "common.cuh"

namespace gb {

__device__ __forceinline__ float ewarp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename T> __device__ __forceinline__ float ld_f32(const T* p);
template <> __device__ __forceinline__ float ld_f32<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ float round_to(float x);
template <> __device__ __forceinline__ float round_to<float>(float x) { return x; }
template <> __device__ __forceinline__ float round_to<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ void load8(const float* p, float (&x)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&x)[8]) {
  const uint4 w = *reinterpret_cast<const uint4*>(p);
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    x[2 * e] = __uint_as_float(ww[e] << 16);
    x[2 * e + 1] = __uint_as_float(ww[e] & 0xffff0000u);
  }
}
__device__ __forceinline__ void store8(float* p, const float (&x)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&x)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
    w[e] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// ---------------------------------------------------------------- dot product
__global__ void emb_chain_val_kernel(const long long* __restrict__ ids_val, long long n_tok, int vocab,
                                     int* __restrict__ head, int* __restrict__ next, int* __restrict__ cnt,
                                     int* __restrict__ err) {
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < n_tok;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long id = ids_val[j];
    if (id >= 0 && id < vocab) {
      next[j] = atomicExch(&head[id], static_cast<int>(j));
      if (cnt != nullptr) atomicAdd(&cnt[id], 1);
    } else {            // the reference's index_add_ raises here; skipped and reported through the error word
      next[j] = -1;
      atomicExch(err, kErrBadIndex);
    }
  }
}

// Ids that many validation tokens share (padding, separators, position ids with a large validation
// batch) would make every train token with that id walk a long chain.  For the `cap` most ... first
// ids whose chain is longer than `threshold`, the validation rows are summed once per (id,
// validation sample) into R[slot][v][d] (float32); a train token then takes n_val dot products
// against R instead of walking the chain.  cnt[id] is overwritten with -(slot + 1) for such ids.
__global__ void emb_hot_assign_kernel(int* __restrict__ cnt, int vocab, int threshold, int cap,
                                      int* __restrict__ n_hot) {
  for (int id = blockIdx.x * blockDim.x + threadIdx.x; id < vocab; id += gridDim.x * blockDim.x) {
    if (cnt[id] > threshold) {
      const int h = atomicAdd(n_hot, 1);
      if (h < cap) cnt[id] = -(h + 1);
    }
  }
}

// one warp per validation token: rows of hot ids are added into R[slot][v]
template <typename T>
__global__ void __launch_bounds__(256)
emb_hot_reduce_kernel(const long long* __restrict__ ids_val, const T* __restrict__ Gval, long long n_tok,
                      long long Tn, int d, int n_val, int vocab, const int* __restrict__ cnt,
                      float* __restrict__ R) {
  const int lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * 8;
  for (long long j = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); j < n_tok; j += warps) {
    const long long id = ids_val[j];
    if (id < 0 || id >= vocab) continue;
    const int c = cnt[id];
    if (c >= 0) continue;
    float* dst = R + (static_cast<long long>(-c - 1) * n_val + j / Tn) * d;
    const T* row = Gval + j * d;
    for (int f = lane; f < d; f += 32) atomicAdd(dst + f, ld_f32<T>(row + f));
  }
}

// grid (token blocks of one sample, n_train); 8 warps, each walks kTokPerWarp tokens
template <typename T>
__global__ void __launch_bounds__(256)
emb_dot_kernel(const long long* __restrict__ ids, const T* __restrict__ G, int n_train, int n_val,
               long long Tn, int d, int vocab, const int* __restrict__ head,
               const int* __restrict__ next, const int* __restrict__ cnt, const float* __restrict__ R,
               float scale, float* __restrict__ M, int tok_per_block, int* __restrict__ err) {
  extern __shared__ float s_acc[];   // [n_val]
  const int b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int v = threadIdx.x; v < n_val; v += blockDim.x) s_acc[v] = 0.f;
  __syncthreads();
  const long long t_begin = static_cast<long long>(blockIdx.x) * tok_per_block;
  long long t_end = t_begin + tok_per_block;
  if (t_end > Tn) t_end = Tn;
  const T* Gval = G + static_cast<long long>(n_train) * Tn * d;
  const bool vec = (d % 8 == 0) && ((reinterpret_cast<uintptr_t>(G) & 15u) == 0);
  for (long long t = t_begin + warp; t < t_end; t += 8) {
    const long long id = ids[static_cast<long long>(b) * Tn + t];
    if (id < 0 || id >= vocab) {
      if (lane == 0) atomicExch(err, kErrBadIndex);
      continue;
    }
    int j = head[id];
    const T* row = G + (static_cast<long long>(b) * Tn + t) * d;
    const int c = (cnt != nullptr) ? cnt[id] : 0;
    if (c < 0) {
      // an id shared by many validation tokens: one dot product per validation sample against the
      // pre-summed rows
      const float* Rh = R + static_cast<long long>(-c - 1) * n_val * d;
      for (int v = 0; v < n_val; ++v) {
        const float* rv = Rh + static_cast<long long>(v) * d;
        float s = 0.f;
        for (int f = lane; f < d; f += 32) s = fmaf(ld_f32<T>(row + f), rv[f], s);
        s = ewarp_sum(s);
        if (lane == 0 && s != 0.f) atomicAdd(&s_acc[v], s);
      }
      continue;
    }
    while (j >= 0) {
      const T* vrow = Gval + static_cast<long long>(j) * d;
      float s = 0.f;
      if (vec && sizeof(T) == 2) {
        for (int f = lane * 8; f < d; f += 256) {
          const uint4 x = *reinterpret_cast<const uint4*>(row + f);
          const uint4 y = *reinterpret_cast<const uint4*>(vrow + f);
          const uint32_t xx[4] = {x.x, x.y, x.z, x.w}, yy[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s = fmaf(__uint_as_float(xx[e] << 16), __uint_as_float(yy[e] << 16), s);
            s = fmaf(__uint_as_float(xx[e] & 0xffff0000u), __uint_as_float(yy[e] & 0xffff0000u), s);
          }
        }
      } else {
        for (int f = lane; f < d; f += 32) s = fmaf(ld_f32<T>(row + f), ld_f32<T>(vrow + f), s);
      }
      s = ewarp_sum(s);
      if (lane == 0) atomicAdd(&s_acc[j / Tn], s);
      j = next[j];
    }
  }
  __syncthreads();
  for (int v = threadIdx.x; v < n_val; v += blockDim.x) {
    const float s = s_acc[v];
    if (s != 0.f) atomicAdd(&M[static_cast<long long>(v) * n_train + b], s * scale);
  }
}

// ---------------------------------------------------------------- train gradient
__global__ void emb_count_kernel(const long long* __restrict__ ids, long long n_tok, int vocab,
                                 int* __restrict__ counts, int* __restrict__ err) {
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < n_tok;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long id = ids[j];
    if (id >= 0 && id < vocab) atomicAdd(&counts[id], 1);
    else atomicExch(err, kErrBadIndex);
  }
}

constexpr int kEmbSmallBucket = 32;      // buckets up to this size are sorted and summed by one warp

// Exclusive scan of counts[0..vocab) into offsets (single block of 1024 threads; tiles of 4096 ids,
// four consecutive ids per thread, the next tile's loads issued before this tile is scanned), and
// the list of rows with more than kEmbSmallBucket tokens for emb_big_bucket_kernel.
__global__ void __launch_bounds__(1024)
emb_scan_kernel(const int* __restrict__ counts, int vocab, int* __restrict__ offsets, int* __restrict__ big,
                int* __restrict__ n_big) {
  __shared__ int s_warp[2][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  auto load4 = [&](int base, int (&c)[4]) {
#pragma unroll
    for (int e = 0; e < 4; ++e) c[e] = (base + e < vocab) ? counts[base + e] : 0;
  };
  int carry = 0, cur[4], nxt[4];
  load4(threadIdx.x * 4, cur);
  int buf = 0;
  for (int tile = 0; tile < vocab; tile += 4096, buf ^= 1) {
    const int base = tile + threadIdx.x * 4;
    load4(base + 4096, nxt);
    const int total = cur[0] + cur[1] + cur[2] + cur[3];
    int x = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) s_warp[buf][warp] = x;
    __syncthreads();
    // every warp scans the 32 warp totals itself (one barrier per tile; the two buffers alternate)
    int w = s_warp[buf][lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += y;
    }
    const int tile_total = __shfl_sync(0xffffffffu, w, 31);
    const int warp_off = __shfl_sync(0xffffffffu, w, (warp + 31) & 31);
    int run = carry + (warp == 0 ? 0 : warp_off) + x - total;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (base + e < vocab) {
        offsets[base + e] = run;
        if (cur[e] > kEmbSmallBucket) big[atomicAdd(n_big, 1)] = base + e;
      }
      run += cur[e];
      cur[e] = nxt[e];
    }
    carry += tile_total;
  }
  if (threadIdx.x == 0) offsets[vocab] = carry;
}

__global__ void emb_fill_kernel(const long long* __restrict__ ids, long long n_tok, int vocab,
                                const int* __restrict__ offsets, int* __restrict__ cursor,
                                int* __restrict__ perm) {
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < n_tok;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long id = ids[j];
    if (id >= 0 && id < vocab) {
      const int pos = atomicAdd(&cursor[id], 1);
      perm[offsets[id] + pos] = static_cast<int>(j);
    }
  }
}

// Shared pieces of the two segment-sum kernels.  A thread owns 8 consecutive features.
template <typename T>
__device__ __forceinline__ void emb_load_row(const T* __restrict__ G, int j, int d, int f, bool vec, float (&x)[8]) {
  const T* row = G + static_cast<long long>(j) * d + f;
  if (vec) {
    if (f < d) {
      load8(row, x);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = 0.f;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = (f + e < d) ? ld_f32<T>(row + e) : 0.f;
  }
}
// no fma contraction: product and sum are rounded separately, as the reference does
template <typename T>
__device__ __forceinline__ void emb_accumulate(const float (&x)[8], float pre_scale, float (&acc)[8]) {
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = __fadd_rn(acc[e], round_to<T>(__fmul_rn(x[e], pre_scale)));
}
template <typename T>
__device__ __forceinline__ void emb_store_row(T* __restrict__ out, int k, int d, int f, bool vec, const float (&acc)[8],
                                              float divisor, int accumulate) {
  T* dst = out + static_cast<long long>(k) * d + f;
  float o[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    o[e] = round_to<T>(__fdiv_rn(round_to<T>(acc[e]), divisor));
    if (accumulate && f + e < d) o[e] = round_to<T>(__fadd_rn(ld_f32<T>(dst + e), o[e]));
  }
  if (vec) {
    if (f < d) store8(dst, o);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (f + e < d) dst[e] = from_f32<T>(o[e]);
  }
}

// Eight consecutive features of a row as loaded (16 bytes of bf16, 32 bytes of float32)
template <typename T> struct EmbRaw;
template <> struct EmbRaw<__nv_bfloat16> {
  using type = uint4;
  static __device__ __forceinline__ uint4 load(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ uint4 zero() { return make_uint4(0u, 0u, 0u, 0u); }
  static __device__ __forceinline__ void unpack(const uint4& w, float (&x)[8]) {
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      x[2 * e] = __uint_as_float(ww[e] << 16);
      x[2 * e + 1] = __uint_as_float(ww[e] & 0xffff0000u);
    }
  }
};
struct EmbFloat8 { float4 a, b; };
template <> struct EmbRaw<float> {
  using type = EmbFloat8;
  static __device__ __forceinline__ EmbFloat8 load(const float* p) {
    EmbFloat8 r;
    r.a = *reinterpret_cast<const float4*>(p);
    r.b = *reinterpret_cast<const float4*>(p + 4);
    return r;
  }
  static __device__ __forceinline__ EmbFloat8 zero() {
    EmbFloat8 r;
    r.a = make_float4(0.f, 0.f, 0.f, 0.f);
    r.b = r.a;
    return r;
  }
  static __device__ __forceinline__ void unpack(const EmbFloat8& w, float (&x)[8]) {
    x[0] = w.a.x; x[1] = w.a.y; x[2] = w.a.z; x[3] = w.a.w; x[4] = w.b.x; x[5] = w.b.y; x[6] = w.b.z; x[7] = w.b.w;
  }
};

// one warp per table row: ascending-order float32 segment sum, dtype rounding as the reference.
// Rows with more than kEmbSmallBucket tokens are left to emb_big_bucket_kernel.  The work of a
// row is the list of (256-feature step, token) units, step-major; the loads of eight units are
// issued before their rows are added in order, so a row with one or two tokens has all its loads
// in flight at once.
template <typename T>
__global__ void __launch_bounds__(256, 3)
emb_segsum_kernel(const T* __restrict__ G, int d, int vocab, const int* __restrict__ offsets,
                  const int* __restrict__ perm, float pre_scale, float divisor, int accumulate,
                  T* __restrict__ out) {
  const int k = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (k >= vocab) return;
  const int off = offsets[k];
  const int cnt = offsets[k + 1] - off;
  if (cnt > kEmbSmallBucket) return;
  const bool vec = (d % 8 == 0) && ((reinterpret_cast<uintptr_t>(G) & 15u) == 0) &&
                   ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
  const int steps = (d + 255) / 256;
  if (cnt == 0) {
    const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < steps; ++c) emb_store_row<T>(out, k, d, c * 256 + lane * 8, vec, zero, divisor, accumulate);
    return;
  }
  int mine = INT_MAX;
  if (lane < cnt) mine = perm[off + lane];
  if (cnt > 1) {
    // bitonic sort of 32 keys across the warp, ascending
#pragma unroll
    for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        const int other = __shfl_xor_sync(0xffffffffu, mine, stride);
        const bool up = ((lane & size) == 0);
        const bool lower = ((lane & stride) == 0);
        const int lo = min(mine, other), hi = max(mine, other);
        mine = (lower == up) ? lo : hi;
      }
    }
  }
  // each lane owns 8 consecutive features of a step (16-byte loads and stores when d % 8 == 0);
  // loaded rows stay packed until they are added (32 registers per batch for either dtype)
  constexpr int kBatch = sizeof(T) == 2 ? 8 : 4;
  const int units = steps * cnt;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  int step = 0, i = 0;                     // unit -> (step, token index), advanced without divisions
  auto finish_unit = [&]() {
    if (++i == cnt) {                      // last token of this step: write the row's 256 features
      emb_store_row<T>(out, k, d, step * 256 + lane * 8, vec, acc, divisor, accumulate);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      i = 0;
      ++step;
    }
  };
  if (!vec) {                              // odd feature counts: one unit at a time
    for (int u = 0; u < units; ++u) {
      float x[8];
      emb_load_row<T>(G, __shfl_sync(0xffffffffu, mine, i), d, step * 256 + lane * 8, false, x);
      emb_accumulate<T>(x, pre_scale, acc);
      finish_unit();
    }
    return;
  }
  using Raw = typename EmbRaw<T>::type;
  for (int u0 = 0; u0 < units; u0 += kBatch) {
    Raw x[kBatch];
    {
      int c = step, ii = i;
#pragma unroll
      for (int r = 0; r < kBatch; ++r) {
        const int j = __shfl_sync(0xffffffffu, mine, ii & 31);
        const int f = c * 256 + lane * 8;
        if (u0 + r < units && f < d) x[r] = EmbRaw<T>::load(G + static_cast<long long>(j) * d + f);
        else x[r] = EmbRaw<T>::zero();
        if (++ii == cnt) { ii = 0; ++c; }
      }
    }
#pragma unroll
    for (int r = 0; r < kBatch; ++r) {
      if (u0 + r < units) {
        float xf[8];
        EmbRaw<T>::unpack(x[r], xf);
        emb_accumulate<T>(xf, pre_scale, acc);
        finish_unit();
      }
    }
  }
}

// Rows that many tokens share (padding, separators, position ids of a large batch).  The list of
// such rows is made by emb_scan_kernel; one CTA per listed row first sorts the row's token
// list into ascending order -- a bitonic network whose comparators all point the same way, so
// entries past the end of the list act as +infinity without being stored; in shared memory up to
// `smem_cap` entries, in place in global memory beyond -- and then sums the rows in that order.
// The sum itself is sequential per feature (float addition in the CPU's order), so the loads of
// the next eight rows are issued before the current eight are added.
__device__ __forceinline__ void emb_bitonic_ascending(int* keys, int cnt, int n2, int tid, int nthreads) {
  for (int k = 2; k <= n2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      // the first stage of every merge pairs i with its mirror image inside the block of k
      for (int i = tid; i < n2; i += nthreads) {
        const int l = (j == (k >> 1)) ? (i ^ (k - 1)) : (i ^ j);
        if (l > i && l < cnt) {
          const int a = keys[i], b = keys[l];
          if (a > b) { keys[i] = b; keys[l] = a; }
        }
      }
      __syncthreads();
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
emb_big_bucket_kernel(const T* __restrict__ G, int d, const int* __restrict__ offsets, int* __restrict__ perm,
                      const int* __restrict__ big, const int* __restrict__ n_big, int smem_cap,
                      float pre_scale, float divisor, int accumulate, T* __restrict__ out) {
  extern __shared__ int s_keys[];
  const int tid = threadIdx.x;
  const int total = *n_big;
  const bool vec = (d % 8 == 0) && ((reinterpret_cast<uintptr_t>(G) & 15u) == 0) &&
                   ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
  for (int bi = blockIdx.x; bi < total; bi += gridDim.x) {
    const int k = big[bi];
    const int off = offsets[k];
    const int cnt = offsets[k + 1] - off;
    int n2 = 64;
    while (n2 < cnt) n2 <<= 1;
    const int* keys;
    __syncthreads();                      // the previous row's readers are done with s_keys
    if (cnt <= smem_cap) {
      for (int i = tid; i < cnt; i += blockDim.x) s_keys[i] = perm[off + i];
      __syncthreads();
      emb_bitonic_ascending(s_keys, cnt, n2, tid, blockDim.x);
      keys = s_keys;
    } else {
      __threadfence_block();
      emb_bitonic_ascending(perm + off, cnt, n2, tid, blockDim.x);   // in place; the CTA owns this range
      keys = perm + off;
    }
    for (int f = tid * 8; f < d; f += blockDim.x * 8) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float cur[8][8], nxt[8][8];
      auto fetch = [&](int i0, float (&buf)[8][8]) {
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (i0 + r < cnt) emb_load_row<T>(G, keys[i0 + r], d, f, vec, buf[r]);
      };
      fetch(0, cur);
      for (int i0 = 0; i0 < cnt; i0 += 8) {
        fetch(i0 + 8, nxt);
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (i0 + r < cnt) emb_accumulate<T>(cur[r], pre_scale, acc);
#pragma unroll
        for (int r = 0; r < 8; ++r)
#pragma unroll
          for (int e = 0; e < 8; ++e) cur[r][e] = nxt[r][e];
      }
      emb_store_row<T>(out, k, d, f, vec, acc, divisor, accumulate);
    }
  }
}

static inline long long up256(long long x) { return (x + 255) / 256 * 256; }

}  // namespace gb

using namespace gb;

// head [vocab] + next [n_val * T]: the least a caller must provide.  With the full size below the
// repeated-id path is enabled as well: cnt [vocab], a counter, and R [kEmbHotCap, n_val, d] float32.
constexpr int kEmbHotCap = 256;
static long long emb_dot_min_bytes(int n_val, long long T, int vocab) {
  return up256(4ll * vocab) + up256(4ll * n_val * T);
}
extern "C" long long ghost_embedding_dot_workspace_bytes_for(int n_val, long long T, int vocab, int d) {
  return emb_dot_min_bytes(n_val, T, vocab) + up256(4ll * vocab) + 256 +
         up256(4ll * kEmbHotCap * static_cast<long long>(n_val) * d);
}
extern "C" long long ghost_embedding_dot_workspace_bytes(int n_val, long long T, int vocab) {
  return emb_dot_min_bytes(n_val, T, vocab);
}

extern "C" int ghost_embedding_dot(const long long* ids, const void* G, int is_f32, int n_train, int n_val,
                                   long long T, int d, int vocab, float scale, float* M_out, void* ws,
                                   long long ws_bytes, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(ids && G && M_out && ws, "ghost_embedding_dot: null pointer");
  GB_REQUIRE(n_train > 0, "No training samples to compute dot product, check batch sizes.");
  GB_REQUIRE(n_val > 0 && T > 0 && d > 0 && vocab > 0, "ghost_embedding_dot: bad dimensions");
  GB_REQUIRE(static_cast<long long>(n_val) * T < INT_MAX && n_train <= 65535, "ghost_embedding_dot: too many tokens");
  GB_REQUIRE(n_val <= 8192, "ghost_embedding_dot: at most 8192 validation samples");
  GB_REQUIRE(ws_bytes >= ghost_embedding_dot_workspace_bytes(n_val, T, vocab), "ghost_embedding_dot: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* head = static_cast<int*>(ws);
  int* next = reinterpret_cast<int*>(static_cast<uint8_t*>(ws) + up256(4ll * vocab));
  const long long n_vtok = static_cast<long long>(n_val) * T;
  // the repeated-id path needs the larger workspace (ghost_embedding_dot_workspace_bytes_for)
  const bool hot = ws_bytes >= ghost_embedding_dot_workspace_bytes_for(n_val, T, vocab, d);
  uint8_t* extra = static_cast<uint8_t*>(ws) + emb_dot_min_bytes(n_val, T, vocab);
  int* cnt = hot ? reinterpret_cast<int*>(extra) : nullptr;
  int* n_hot = hot ? reinterpret_cast<int*>(extra + up256(4ll * vocab)) : nullptr;
  float* R = hot ? reinterpret_cast<float*>(extra + up256(4ll * vocab) + 256) : nullptr;
  if (hot) GB_CUDA_OK(cudaMemsetAsync(cnt, 0, up256(4ll * vocab) + 256, st));
  GB_CUDA_OK(cudaMemsetAsync(head, 0xFF, 4ull * vocab, st));
  GB_CUDA_OK(cudaMemsetAsync(M_out, 0, sizeof(float) * static_cast<size_t>(n_val) * n_train, st));
  int blocks = static_cast<int>((n_vtok + 255) / 256);
  if (blocks > ds->sm_count * 8) blocks = ds->sm_count * 8;
  emb_chain_val_kernel<<<blocks, 256, 0, st>>>(ids + static_cast<long long>(n_train) * T, n_vtok, vocab, head, next, cnt, ds->err_word);
  count_launch();
  int rc = post_launch("emb_chain_val_kernel");
  if (rc != GHOST_OK) return rc;
  if (hot) {
    // chains longer than four dot products per validation sample are worth summing up front
    const int threshold = 4 * n_val > 16 ? 4 * n_val : 16;
    if (n_vtok > threshold) {
      GB_CUDA_OK(cudaMemsetAsync(R, 0, 4ull * kEmbHotCap * static_cast<size_t>(n_val) * d, st));
      int vb = ceil_div(vocab, 256);
      if (vb > ds->sm_count * 4) vb = ds->sm_count * 4;
      emb_hot_assign_kernel<<<vb, 256, 0, st>>>(cnt, vocab, threshold, kEmbHotCap, n_hot);
      int rb = static_cast<int>((n_vtok + 7) / 8);
      if (rb > ds->sm_count * 8) rb = ds->sm_count * 8;
      const long long* ids_val = ids + static_cast<long long>(n_train) * T;
      if (is_f32)
        emb_hot_reduce_kernel<float><<<rb, 256, 0, st>>>(ids_val, static_cast<const float*>(G) + static_cast<long long>(n_train) * T * d, n_vtok, T, d, n_val, vocab, cnt, R);
      else
        emb_hot_reduce_kernel<__nv_bfloat16><<<rb, 256, 0, st>>>(ids_val, static_cast<const __nv_bfloat16*>(G) + static_cast<long long>(n_train) * T * d, n_vtok, T, d, n_val, vocab, cnt, R);
      count_launch(2);
      if ((rc = post_launch("emb_hot_reduce_kernel")) != GHOST_OK) return rc;
    }
  }
  const int tok_per_block = 64;
  dim3 grid(ceil_div(T, tok_per_block), n_train);
  const size_t smem = sizeof(float) * n_val;
  if (is_f32)
    emb_dot_kernel<float><<<grid, 256, smem, st>>>(ids, static_cast<const float*>(G), n_train, n_val, T, d, vocab, head, next, cnt, R, scale, M_out, tok_per_block, ds->err_word);
  else
    emb_dot_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(ids, static_cast<const __nv_bfloat16*>(G), n_train, n_val, T, d, vocab, head, next, cnt, R, scale, M_out, tok_per_block, ds->err_word);
  count_launch();
  return post_launch("emb_dot_kernel");
}

// counts, offsets, cursor ([vocab + 1] each), the token permutation, and the list of rows with more
// than kEmbSmallBucket tokens (its counter in front)
static long long emb_big_list_bytes(long long n_tok) { return up256(4ll * (n_tok / (kEmbSmallBucket + 1) + 2)); }
extern "C" long long ghost_embedding_wgrad_workspace_bytes(int n_train, long long T, int vocab) {
  return 3 * up256(4ll * (vocab + 1)) + up256(4ll * n_train * T) + emb_big_list_bytes(static_cast<long long>(n_train) * T);
}

extern "C" int ghost_embedding_wgrad(const long long* ids, const void* G, int is_f32, int n_train, long long T,
                                     int d, int vocab, float pre_scale, float divisor, int accumulate,
                                     void* out, void* ws, long long ws_bytes, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(ids && G && out && ws, "ghost_embedding_wgrad: null pointer");
  GB_REQUIRE(n_train > 0 && T > 0 && d > 0 && vocab > 0, "ghost_embedding_wgrad: bad dimensions");
  GB_REQUIRE(static_cast<long long>(n_train) * T < INT_MAX, "ghost_embedding_wgrad: too many tokens");
  GB_REQUIRE(divisor != 0.f, "ghost_embedding_wgrad: divisor must be non-zero");
  GB_REQUIRE(ws_bytes >= ghost_embedding_wgrad_workspace_bytes(n_train, T, vocab), "ghost_embedding_wgrad: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* w = static_cast<uint8_t*>(ws);
  const long long seg = up256(4ll * (vocab + 1));
  const long long n_tok = static_cast<long long>(n_train) * T;
  // counts, cursor and the big-row counter sit next to each other: one memset clears them
  int* counts = reinterpret_cast<int*>(w);
  int* cursor = reinterpret_cast<int*>(w + seg);
  int* n_big = reinterpret_cast<int*>(w + 2 * seg);
  int* big = n_big + 1;
  int* offsets = reinterpret_cast<int*>(w + 2 * seg + emb_big_list_bytes(n_tok));
  int* perm = reinterpret_cast<int*>(w + 3 * seg + emb_big_list_bytes(n_tok));
  GB_CUDA_OK(cudaMemsetAsync(counts, 0, 2 * seg + 4, st));
  int blocks = static_cast<int>((n_tok + 255) / 256);
  if (blocks > ds->sm_count * 8) blocks = ds->sm_count * 8;
  emb_count_kernel<<<blocks, 256, 0, st>>>(ids, n_tok, vocab, counts, ds->err_word);
  emb_scan_kernel<<<1, 1024, 0, st>>>(counts, vocab, offsets, big, n_big);
  emb_fill_kernel<<<blocks, 256, 0, st>>>(ids, n_tok, vocab, offsets, cursor, perm);
  // rows shared by many tokens: sorted in up to 128 KB of shared memory (32768 tokens), else in place
  constexpr int kSmemCap = 32768;
  static bool attr_set[64] = {};
  if (!attr_set[ds->device]) {
    GB_CUDA_OK(cudaFuncSetAttribute(emb_big_bucket_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemCap * 4));
    GB_CUDA_OK(cudaFuncSetAttribute(emb_big_bucket_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemCap * 4));
    attr_set[ds->device] = true;
  }
  long long big_max = n_tok / (kEmbSmallBucket + 1) + 1;
  const int big_blocks = static_cast<int>(big_max < ds->sm_count ? big_max : ds->sm_count);
  if (is_f32) {
    emb_segsum_kernel<float><<<ceil_div(vocab, 8), 256, 0, st>>>(static_cast<const float*>(G), d, vocab, offsets, perm, pre_scale, divisor, accumulate, static_cast<float*>(out));
    emb_big_bucket_kernel<float><<<big_blocks, 256, kSmemCap * 4, st>>>(static_cast<const float*>(G), d, offsets, perm, big, n_big, kSmemCap, pre_scale, divisor, accumulate, static_cast<float*>(out));
  } else {
    emb_segsum_kernel<__nv_bfloat16><<<ceil_div(vocab, 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(G), d, vocab, offsets, perm, pre_scale, divisor, accumulate, static_cast<__nv_bfloat16*>(out));
    emb_big_bucket_kernel<__nv_bfloat16><<<big_blocks, 256, kSmemCap * 4, st>>>(static_cast<const __nv_bfloat16*>(G), d, offsets, perm, big, n_big, kSmemCap, pre_scale, divisor, accumulate, static_cast<__nv_bfloat16*>(out));
  }
  count_launch(5);
  return post_launch("ghost_embedding_wgrad");
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of ghost_embedding_dot.
//
// Who needs it: callers that are not allowed to obtain device memory when the hook fires.  Two real
// cases: a process whose device memory is owned up front by a fixed-size pool (an inference or
// data-valuation service with a hard memory budget, where a late cudaMalloc can fail or stall every
// stream while the driver synchronises), and code that runs inside another component's critical
// section (an allocator callback, a communication progress thread) where calling back into any
// allocator, torch's included, would deadlock.  Such callers can still hand over their inputs and
// the output matrix, but they have nowhere to get the id-chain tables from.
//
// The tables therefore live in the library image itself: one file-scope __device__ array per GPU
// that loads the library (kEmbStaticBytes, held until the process exits).  Limits follow from its
// size: vocab <= 131072 and n_val * T <= 131072.  Larger problems are rejected; use
// ghost_embedding_dot with a caller-provided workspace for those.
//
// The array's name is a host-side handle, not a device address, so the device address is looked up
// with cudaGetSymbolAddress the first time the entry point runs on a device (with that device
// current) and cached.  That first call should happen before any stream capture begins.  The
// tables keep whatever the previous call left: every call re-initialises the head table and
// rewrites the whole next-table range it uses before reading it.  All calls on one GPU share the
// one array, so two calls whose kernels can overlap (different streams, no ordering) race; keep
// calls to this entry point on one stream or order them with events.
// ------------------------------------------------------------------------------------------------
namespace gb {
constexpr int kEmbStaticMaxVocab = 131072;
constexpr long long kEmbStaticMaxValTokens = 131072;
constexpr long long kEmbStaticBytes = 4ll * kEmbStaticMaxVocab + 4ll * kEmbStaticMaxValTokens;   // 1 MiB
static __device__ __align__(256) unsigned char g_emb_static_scratch[kEmbStaticBytes];

static int emb_static_scratch(void** out) {
  static std::mutex mu;
  static void* ptrs[64] = {};
  int dev = -1;
  GB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(GHOST_ERR_INVALID, "unsupported device ordinal %d", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    // set-up, once per device, with that device current
    GB_CUDA_OK(cudaGetSymbolAddress(&p, g_emb_static_scratch));
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return GHOST_OK;
}
}  // namespace gb

extern "C" int ghost_embedding_dot_noalloc(const long long* ids, const void* G, int is_f32, int n_train,
                                           int n_val, long long T, int d, int vocab, float scale,
                                           float* M_out, void* stream) {
  if (!device_state()) return GHOST_ERR_DEVICE;
  GB_REQUIRE(vocab > 0 && vocab <= kEmbStaticMaxVocab,
             "ghost_embedding_dot_noalloc: vocab %d exceeds the built-in scratch (max %d); use "
             "ghost_embedding_dot with a caller workspace", vocab, kEmbStaticMaxVocab);
  GB_REQUIRE(n_val > 0 && T > 0 && static_cast<long long>(n_val) * T <= kEmbStaticMaxValTokens,
             "ghost_embedding_dot_noalloc: n_val * T = %lld exceeds the built-in scratch (max %lld); use "
             "ghost_embedding_dot with a caller workspace", static_cast<long long>(n_val) * T,
             kEmbStaticMaxValTokens);
  void* scratch = nullptr;
  int rc = emb_static_scratch(&scratch);
  if (rc != GHOST_OK) return rc;
  // same kernels as ghost_embedding_dot; the head table is cleared and the used part of the next
  // table rewritten on every call, so stale contents of the shared array are never read
  return ghost_embedding_dot(ids, G, is_f32, n_train, n_val, T, d, vocab, scale, M_out, scratch,
                             kEmbStaticBytes, stream);
}
