// tile_dot: second half of the per-sample-gradient path.
//
// xty_gemm (kEpiStoreTiles) leaves the per-sample weight-gradient tiles of the validation samples
// (V) and of a group of train samples (W) in a workspace, tile-major.  This kernel streams both
// once and produces
//     M[v, b]  += scale * sum_k V[v][k] * W[b][k]        (Frobenius products, reference :135)
//     sum[k]   (+)= sum_b W[b][k]                        (the train gradient, reference :168)
// Each warp owns a contiguous range of 64-element chunks of the flattened tile space, so the
// train-gradient sum is a plain read-modify-write (no atomics, deterministic); the 8 x 32 block of
// dot products a warp accumulates is reduced with shuffles and added to M once per warp.
// Bandwidth-bound: every workspace byte is read once per (8 validation x 32 train) block.
#include "common.cuh"

namespace gb {

// 8 consecutive stored elements, kept packed in registers until they are used
template <typename T> struct Pack8;
template <> struct Pack8<__nv_bfloat16> {
  uint4 w;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { w = __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void zero() { w = make_uint4(0u, 0u, 0u, 0u); }
  __device__ __forceinline__ void unpack(float (&x)[8]) const {
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      x[2 * e] = __uint_as_float(ww[e] << 16);
      x[2 * e + 1] = __uint_as_float(ww[e] & 0xffff0000u);
    }
  }
};
template <> struct Pack8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = __ldg(reinterpret_cast<const float4*>(p));
    b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void zero() { a = make_float4(0.f, 0.f, 0.f, 0.f); b = a; }
  __device__ __forceinline__ void unpack(float (&x)[8]) const {
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
};

struct TileDotParams {
  const void* V;          // [tiles][n_val][32768]
  const void* W;          // [tiles][n_grp][32768]
  long long chunks;       // tiles * 1024 (32-element chunks)
  long long chunks_per_warp;
  int n_val, n_grp;       // validation samples, train samples in this group
  int b0, n_train;        // first train sample of the group, total train samples (M row pitch)
  float scale;
  float* M;               // [n_val, n_train]
  float* sum;             // [tiles * 32768] fp32 or null
  int sum_init;           // 1: this group overwrites sum, 0: it accumulates
};

constexpr int kTileElems = 128 * 256;
constexpr int kChunk = 32;                           // elements per warp step (4 lanes x 8)
constexpr int kChunksPerTile = kTileElems / kChunk;  // 1024

// Lane layout: kg = lane & 3 picks one 8-element vector of the 32-element chunk, bg = lane >> 2
// picks 4 of the 32 train samples of the block.  A thread accumulates an 8 (validation) x 4
// (train) block of dot products over its vectors.
template <typename T>
__global__ void __launch_bounds__(256, sizeof(T) == 2 ? 2 : 1)
tile_dot_kernel(const TileDotParams p) {
  const int lane = threadIdx.x & 31;
  const int kg = lane & 3;
  const int bg = lane >> 2;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long c_begin = warp * p.chunks_per_warp;
  long long c_end = c_begin + p.chunks_per_warp;
  if (c_end > p.chunks) c_end = p.chunks;
  if (c_begin >= c_end) return;
  const T* V = static_cast<const T*>(p.V);
  const T* W = static_cast<const T*>(p.W);

  for (int j0 = 0; j0 < p.n_grp; j0 += 32) {          // 32-train-sample blocks
    for (int v0 = 0; v0 < p.n_val; v0 += 8) {          // 8-validation-sample blocks
      float acc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[i][q] = 0.f;
      const bool do_sum = (v0 == 0) && (p.sum != nullptr);
#pragma unroll 1
      for (long long c = c_begin; c < c_end; ++c) {
        const long long tile = c / kChunksPerTile;
        const int e = static_cast<int>(c % kChunksPerTile) * kChunk + kg * 8;
        // phase 1: every load of the chunk is issued before any arithmetic (12 independent
        // 16-byte requests per thread in flight)
        Pack8<T> pw[4], pv[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int b = j0 + bg * 4 + q;
          if (b < p.n_grp) pw[q].load(W + (tile * p.n_grp + b) * kTileElems + e);
          else pw[q].zero();
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int v = v0 + i;
          if (v < p.n_val) pv[i].load(V + (tile * p.n_val + v) * kTileElems + e);
          else pv[i].zero();
        }
        // phase 2: unpack and accumulate
        float w[4][8];
        float s[8];
#pragma unroll
        for (int x = 0; x < 8; ++x) s[x] = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          pw[q].unpack(w[q]);
#pragma unroll
          for (int x = 0; x < 8; ++x) s[x] += w[q][x];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float vv[8];
          pv[i].unpack(vv);
#pragma unroll
          for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int x = 0; x < 8; ++x) acc[i][q] = fmaf(vv[x], w[q][x], acc[i][q]);
        }
        if (do_sum) {
          // sum over the eight 4-sample groups of the warp, then one 32-byte update per kg lane
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            s[x] += __shfl_xor_sync(0xffffffffu, s[x], 4);
            s[x] += __shfl_xor_sync(0xffffffffu, s[x], 8);
            s[x] += __shfl_xor_sync(0xffffffffu, s[x], 16);
          }
          if (bg == 0) {
            float4* dst = reinterpret_cast<float4*>(p.sum + c * kChunk + kg * 8);
            float4 a = make_float4(s[0], s[1], s[2], s[3]), b = make_float4(s[4], s[5], s[6], s[7]);
            if (!(p.sum_init && j0 == 0)) {
              const float4 oa = dst[0], ob = dst[1];
              a.x += oa.x; a.y += oa.y; a.z += oa.z; a.w += oa.w;
              b.x += ob.x; b.y += ob.y; b.z += ob.z; b.w += ob.w;
            }
            dst[0] = a;
            dst[1] = b;
          }
        }
      }
      // reduce the 8 x 4 block over the four kg lanes, then one atomic per (v, b)
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float a = acc[i][q];
          a += __shfl_xor_sync(0xffffffffu, a, 1);
          a += __shfl_xor_sync(0xffffffffu, a, 2);
          const int v = v0 + i, b = j0 + bg * 4 + q;
          if (kg == 0 && v < p.n_val && b < p.n_grp && a != 0.f)
            atomicAdd(&p.M[static_cast<long long>(v) * p.n_train + p.b0 + b], a * p.scale);
        }
    }
  }
}

// out[r, c] (= or +=) scale * sum[tile(r, c)][r % 128][c % 256], cast to the parameter dtype
template <typename OutT>
__global__ void tile_sum_finalize_kernel(const float* __restrict__ sum, int n_tiles_n, OutT* __restrict__ out,
                                         int rows, int cols, float scale, int accumulate) {
  const long long n = static_cast<long long>(rows) * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / cols), c = static_cast<int>(i % cols);
    const long long tile = static_cast<long long>(r >> 7) * n_tiles_n + (c >> 8);
    float v = sum[tile * kTileElems + (r & 127) * 256 + (c & 255)] * scale;
    if (accumulate) v += static_cast<float>(out[i]);
    out[i] = static_cast<OutT>(v);
  }
}

int launch_tile_dot(const void* V, const void* W, int is_f32, long long tiles, int n_val, int n_grp, int b0,
                    int n_train, float scale, float* M, float* sum, int sum_init, const DeviceState* ds,
                    cudaStream_t st) {
  TileDotParams p;
  p.V = V; p.W = W;
  p.chunks = tiles * kChunksPerTile;
  p.n_val = n_val; p.n_grp = n_grp; p.b0 = b0; p.n_train = n_train;
  p.scale = scale; p.M = M; p.sum = sum; p.sum_init = sum_init;
  long long warps = static_cast<long long>(ds->sm_count) * 16;      // two 256-thread CTAs per SM
  if (warps > p.chunks) warps = p.chunks;
  p.chunks_per_warp = (p.chunks + warps - 1) / warps;
  warps = (p.chunks + p.chunks_per_warp - 1) / p.chunks_per_warp;
  const int blocks = static_cast<int>((warps + 7) / 8);
  if (is_f32) tile_dot_kernel<float><<<blocks, 256, 0, st>>>(p);
  else tile_dot_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(p);
  count_launch();
  return post_launch("tile_dot_kernel");
}

int launch_tile_sum_finalize(const float* sum, int n_tiles_n, void* out, int out_is_f32, int rows, int cols,
                             float scale, int accumulate, const DeviceState* ds, cudaStream_t st) {
  const long long n = static_cast<long long>(rows) * cols;
  long long blocks = (n + 255) / 256;
  if (blocks > ds->sm_count * 8) blocks = ds->sm_count * 8;
  if (out_is_f32)
    tile_sum_finalize_kernel<float><<<static_cast<int>(blocks), 256, 0, st>>>(sum, n_tiles_n, static_cast<float*>(out), rows, cols, scale, accumulate);
  else
    tile_sum_finalize_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(sum, n_tiles_n, static_cast<__nv_bfloat16*>(out), rows, cols, scale, accumulate);
  count_launch();
  return post_launch("tile_sum_finalize_kernel");
}

}  // namespace gb
