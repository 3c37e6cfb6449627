// Two small kernels on the edges of the GradProj path.
//
//  * gradproj_embedding_kernel: per-sample projected gradient of an embedding table,
//      out[b][o][i] = scale * sum_t (P_o g_bt)[o] * P_i[i, id_bt]
//    (GhostSuite computes it with a Python loop over every token and one .item() host sync per
//    token: ghostEngines/gradProjection/autograd_gradproj.py:167-222).  The out-grad rows are
//    streamed once; P_o g_t for 16 tokens per warp runs on mma.sync with fragments loaded straight
//    from global memory, the k_o x k_i outer-product accumulation over a block of 64 tokens on the
//    CUDA cores out of shared memory, where the gathered rows of P_i^T sit.
//
//  * proj_similarity_kernel: S = scale * P1 P2^T for two blocks of projection rows
//    [n, total_proj_dim] (Examples/ghost_gradproj_lm.py:190-196): a few rows, a very long
//    contraction, bound by streaming both operands once.  The contraction is split over all
//    warps of the grid, 16 x 16 outputs per warp, partial sums added with atomics.
//
// float operands are split into bf16 hi/lo parts in registers (hi*hi + lo*hi + hi*lo).
#include "common.cuh"
#include "mma_sync.cuh"

namespace gb {

// ------------------------------------------------------------------------------------------------
// embedding projection
// ------------------------------------------------------------------------------------------------
struct EmbProjParams {
  const long long* ids;   // [B, T]
  const void* G;          // [B, T, d], row pitch ldg
  long long T, ldg;
  int d, vocab, k_o, k_i;
  const __nv_bfloat16* P_o;   // [k_o, ldp]: bf16(P_o) in columns [0, cp); for float out-grads the
  long long ldp;              // residual P_o - bf16(P_o) in columns [lo_off, lo_off + cp)
  int cp, lo_off;
  const float* PiT;       // [vocab, >= k_i] with row pitch ld_pit: P_i transposed, one row per token id
  long long ld_pit;
  float scale;
  float* out;             // [B, out_stride]; the sample's block starts at its row, o-rows out_ld apart
  long long out_stride;
  int out_ld;
  int* err;
};

static constexpr int kTokBlock = 64;    // tokens per pass of a CTA (4 warps x 16)
static constexpr int kUPitch = 68;      // floats per token row of the projected out-grads (64 + 4)

template <typename GT, int NT, bool VEC>
__global__ void __launch_bounds__(128) gradproj_embedding_kernel(EmbProjParams p) {
  __shared__ __align__(16) float U[kTokBlock * kUPitch];   // [token][o]
  __shared__ __align__(16) float Q[kTokBlock * 64];        // [token][i]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int b = blockIdx.y;
  const GT* Gb = static_cast<const GT*>(p.G) + static_cast<long long>(b) * p.T * p.ldg;
  const long long* idb = p.ids + static_cast<long long>(b) * p.T;
  constexpr bool kSplit = sizeof(GT) == 4;

  // stage-2 ownership: 8 output rows (o) x 4 output columns (i) per thread
  const int to = tid >> 4, ti = tid & 15;
  float acc2[8][4];
#pragma unroll
  for (int r = 0; r < 8; ++r)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc2[r][q] = 0.f;

  const long long n_blocks = (p.T + kTokBlock - 1) / kTokBlock;
  for (long long tb = blockIdx.x; tb < n_blocks; tb += gridDim.x) {
    const long long t0 = tb * kTokBlock + 16 * warp;
    // ---- stage 1: U[16 tokens of this warp][k_o] = G rows x P_o^T --------------------------------
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const bool r0_ok = t0 + g < p.T, r1_ok = t0 + g + 8 < p.T;
    const GT* row0 = Gb + (t0 + g) * p.ldg;
    const GT* row1 = Gb + (t0 + g + 8) * p.ldg;
#pragma unroll 2
    for (int k0 = 0; k0 < p.d; k0 += 16) {
      const long long k = k0 + 4 * c;
      const Quad a0 = load_quad<VEC>(row0, k, p.d, r0_ok);
      const Quad a1 = load_quad<VEC>(row1, k, p.d, r1_ok);
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int o = 8 * j + g;
        const bool o_ok = o < p.k_o;
        const __nv_bfloat16* prow = p.P_o + static_cast<long long>(o) * p.ldp;
        const Quad bh = load_quad<true>(prow, k, p.cp, o_ok);
        mma_16816(acc[j], a0.hi[0], a1.hi[0], a0.hi[1], a1.hi[1], bh.hi[0], bh.hi[1]);
        if (kSplit) {
          mma_16816(acc[j], a0.lo[0], a1.lo[0], a0.lo[1], a1.lo[1], bh.hi[0], bh.hi[1]);
          const Quad bl = load_quad<true>(prow + p.lo_off, k, p.cp, o_ok);
          mma_16816(acc[j], a0.hi[0], a1.hi[0], a0.hi[1], a1.hi[1], bl.hi[0], bl.hi[1]);
        }
      }
    }
    __syncthreads();          // the previous block's stage 2 has finished reading U and Q
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      float* u0 = &U[(16 * warp + g) * kUPitch + 8 * j + 2 * c];
      float* u1 = u0 + 8 * kUPitch;
      u0[0] = acc[j][0]; u0[1] = acc[j][1];
      u1[0] = acc[j][2]; u1[1] = acc[j][3];
    }
    // gathered rows of P_i^T: Q[token][0..k_i) (zero for tokens past the end and for bad ids)
    for (int e = tid; e < kTokBlock * 16; e += 128) {
      const int t = e >> 4, q4 = (e & 15) * 4;
      const long long tt = tb * kTokBlock + t;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tt < p.T && q4 < p.k_i) {
        const long long id = idb[tt];
        if (id >= 0 && id < p.vocab) {
          const float* src = p.PiT + id * p.ld_pit + q4;
          v.x = __ldg(src);
          if (q4 + 1 < p.k_i) v.y = __ldg(src + 1);
          if (q4 + 2 < p.k_i) v.z = __ldg(src + 2);
          if (q4 + 3 < p.k_i) v.w = __ldg(src + 3);
        } else if (q4 == 0) {
          atomicExch(p.err, kErrBadIndex);
        }
      }
      *reinterpret_cast<float4*>(&Q[t * 64 + q4]) = v;
    }
    __syncthreads();
    // ---- stage 2: out[o][i] += sum over the block's tokens of U[t][o] * Q[t][i] ------------------
    if (to < NT) {
#pragma unroll 4
      for (int t = 0; t < kTokBlock; ++t) {
        const float4 ua = *reinterpret_cast<const float4*>(&U[t * kUPitch + 8 * to]);
        const float4 ub = *reinterpret_cast<const float4*>(&U[t * kUPitch + 8 * to + 4]);
        const float4 qv = *reinterpret_cast<const float4*>(&Q[t * 64 + 4 * ti]);
        const float u[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
        const float q[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
        for (int r = 0; r < 8; ++r)
#pragma unroll
          for (int s = 0; s < 4; ++s) acc2[r][s] = fmaf(u[r], q[s], acc2[r][s]);
      }
    }
  }
  if (to < NT) {
    float* ob = p.out + static_cast<long long>(b) * p.out_stride;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int o = 8 * to + r;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const int i = 4 * ti + s;
        if (o < p.k_o && i < p.k_i) atomicAdd(ob + static_cast<long long>(o) * p.out_ld + i, p.scale * acc2[r][s]);
      }
    }
  }
}

template <typename GT, int NT>
static int launch_emb_proj(const EmbProjParams& p, bool vec, dim3 grid, cudaStream_t st) {
  if (vec)
    gradproj_embedding_kernel<GT, NT, true><<<grid, 128, 0, st>>>(p);
  else
    gradproj_embedding_kernel<GT, NT, false><<<grid, 128, 0, st>>>(p);
  count_launch();
  return post_launch("gradproj_embedding_kernel");
}

template <typename GT>
static int dispatch_emb_proj(const EmbProjParams& p, bool vec, dim3 grid, cudaStream_t st) {
  const int nt = (p.k_o + 7) / 8;
  if (nt <= 1) return launch_emb_proj<GT, 1>(p, vec, grid, st);
  if (nt <= 2) return launch_emb_proj<GT, 2>(p, vec, grid, st);
  if (nt <= 4) return launch_emb_proj<GT, 4>(p, vec, grid, st);
  return launch_emb_proj<GT, 8>(p, vec, grid, st);
}

// ------------------------------------------------------------------------------------------------
// similarity of projection rows
// ------------------------------------------------------------------------------------------------
struct SimParams {
  const void* P1;   // [n1, D], row pitch ld1
  const void* P2;   // [n2, D], row pitch ld2
  int n1, n2;
  long long D, ld1, ld2;
  float scale;
  float* S;         // [n1, ld_s]
  long long ld_s;
};

template <typename PT, bool VEC>
__global__ void __launch_bounds__(256) proj_similarity_kernel(SimParams p) {
  __shared__ float part[8][16 * 16];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int i0 = blockIdx.y * 16, j0 = blockIdx.z * 16;
  constexpr bool kSplit = sizeof(PT) == 4;
  const PT* A = static_cast<const PT*>(p.P1);
  const PT* Bm = static_cast<const PT*>(p.P2);
  const bool a0_ok = i0 + g < p.n1, a1_ok = i0 + g + 8 < p.n1;
  const bool b0_ok = j0 + g < p.n2, b1_ok = j0 + g + 8 < p.n2;
  const PT* ar0 = A + static_cast<long long>(i0 + g) * p.ld1;
  const PT* ar1 = A + static_cast<long long>(i0 + g + 8) * p.ld1;
  const PT* br0 = Bm + static_cast<long long>(j0 + g) * p.ld2;
  const PT* br1 = Bm + static_cast<long long>(j0 + g + 8) * p.ld2;

  // every warp of the grid takes one contiguous range of 16-element blocks of the contraction
  const long long nkb = (p.D + 15) / 16;
  const long long warps = static_cast<long long>(gridDim.x) * 8;
  const long long per = (nkb + warps - 1) / warps;
  const long long w = static_cast<long long>(blockIdx.x) * 8 + warp;
  const long long kb_lo = w * per;
  const long long kb_hi = (kb_lo + per < nkb) ? kb_lo + per : nkb;

  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
  for (long long kb = kb_lo; kb < kb_hi; ++kb) {
    const long long k = kb * 16 + 4 * c;
    const Quad a0 = load_quad<VEC>(ar0, k, p.D, a0_ok);
    const Quad a1 = load_quad<VEC>(ar1, k, p.D, a1_ok);
    const Quad b0 = load_quad<VEC>(br0, k, p.D, b0_ok);
    const Quad b1 = load_quad<VEC>(br1, k, p.D, b1_ok);
    mma_16816(acc[0], a0.hi[0], a1.hi[0], a0.hi[1], a1.hi[1], b0.hi[0], b0.hi[1]);
    mma_16816(acc[1], a0.hi[0], a1.hi[0], a0.hi[1], a1.hi[1], b1.hi[0], b1.hi[1]);
    if (kSplit) {
      mma_16816(acc[0], a0.lo[0], a1.lo[0], a0.lo[1], a1.lo[1], b0.hi[0], b0.hi[1]);
      mma_16816(acc[1], a0.lo[0], a1.lo[0], a0.lo[1], a1.lo[1], b1.hi[0], b1.hi[1]);
      mma_16816(acc[0], a0.hi[0], a1.hi[0], a0.hi[1], a1.hi[1], b0.lo[0], b0.lo[1]);
      mma_16816(acc[1], a0.hi[0], a1.hi[0], a0.hi[1], a1.hi[1], b1.lo[0], b1.lo[1]);
    }
  }
  // fragment -> [16][16]: n-tile j covers columns 8j .. 8j+7
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    part[warp][g * 16 + 8 * j + 2 * c] = acc[j][0];
    part[warp][g * 16 + 8 * j + 2 * c + 1] = acc[j][1];
    part[warp][(g + 8) * 16 + 8 * j + 2 * c] = acc[j][2];
    part[warp][(g + 8) * 16 + 8 * j + 2 * c + 1] = acc[j][3];
  }
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int ww = 0; ww < 8; ++ww) s += part[ww][tid];
  const int i = i0 + (tid >> 4), j = j0 + (tid & 15);
  if (i < p.n1 && j < p.n2 && s != 0.f) atomicAdd(p.S + static_cast<long long>(i) * p.ld_s + j, p.scale * s);
}

}  // namespace gb

using namespace gb;

extern "C" int ghost_gradproj_embedding(const long long* ids, const void* G, int g_is_f32, int B, long long T,
                                        int d, long long ldg, const void* P_o, long long ldp_o, int p_cols,
                                        int p_lo_offset, const float* P_i_t, long long ld_pit, int vocab, int k_o,
                                        int k_i, float scale, int accumulate, float* out, long long out_stride,
                                        int out_ld, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(ids && G && P_o && P_i_t && out, "ghost_gradproj_embedding: null pointer");
  GB_REQUIRE(B > 0 && T > 0 && d > 0 && vocab > 0, "ghost_gradproj_embedding: empty dimension");
  GB_REQUIRE(k_o >= 1 && k_o <= 64 && k_i >= 1 && k_i <= 64,
             "ghost_gradproj_embedding: k_o and k_i must be between 1 and 64 (got %d, %d)", k_o, k_i);
  GB_REQUIRE(ldg >= d && ld_pit >= k_i && out_ld >= k_i &&
                 out_stride >= static_cast<long long>(k_o - 1) * out_ld + k_i,
             "ghost_gradproj_embedding: pitch smaller than the row it holds");
  GB_REQUIRE(accumulate || out_ld == k_i,
             "ghost_gradproj_embedding: a block inside wider rows (out_ld > k_i) must be zeroed by the caller "
             "and passed with accumulate = 1");
  GB_REQUIRE(p_cols >= d && p_cols % 8 == 0 && ldp_o % 8 == 0 && ldp_o >= p_cols &&
                 (reinterpret_cast<uintptr_t>(P_o) & 15u) == 0,
             "ghost_gradproj_embedding: P_o must be 16-byte aligned bf16 with columns padded to a multiple of 8");
  GB_REQUIRE(!g_is_f32 || (p_lo_offset % 8 == 0 && p_lo_offset >= p_cols && p_lo_offset + p_cols <= ldp_o),
             "ghost_gradproj_embedding: float out-grads need the residual part of P_o inside its rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!accumulate)
    GB_CUDA_OK(cudaMemset2DAsync(out, static_cast<size_t>(out_stride) * 4, 0, static_cast<size_t>(k_o) * k_i * 4,
                                 static_cast<size_t>(B), st));
  EmbProjParams p = {};
  p.ids = ids; p.G = G; p.T = T; p.ldg = ldg; p.d = d; p.vocab = vocab; p.k_o = k_o; p.k_i = k_i;
  p.P_o = static_cast<const __nv_bfloat16*>(P_o); p.ldp = ldp_o; p.cp = p_cols; p.lo_off = p_lo_offset;
  p.PiT = P_i_t; p.ld_pit = ld_pit; p.scale = scale; p.out = out; p.out_stride = out_stride; p.out_ld = out_ld;
  p.err = ds->err_word;
  const long long n_blocks = (T + kTokBlock - 1) / kTokBlock;
  long long splits = (2ll * ds->sm_count + B - 1) / B;
  if (splits > n_blocks) splits = n_blocks;
  if (splits < 1) splits = 1;
  GB_REQUIRE(B <= 65535, "ghost_gradproj_embedding: more than 65535 samples in one call");
  const dim3 grid(static_cast<unsigned>(splits), static_cast<unsigned>(B), 1);
  const int esize = g_is_f32 ? 4 : 2;
  const bool vec = d % 4 == 0 && ldg % 4 == 0 && (reinterpret_cast<uintptr_t>(G) % (4 * esize)) == 0;
  return g_is_f32 ? dispatch_emb_proj<float>(p, vec, grid, st) : dispatch_emb_proj<__nv_bfloat16>(p, vec, grid, st);
}

extern "C" int ghost_projection_similarity(const void* P1, const void* P2, int is_f32, int n1, int n2, long long D,
                                           long long ld1, long long ld2, float scale, float* S, long long ld_s,
                                           void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(P1 && P2 && S, "ghost_projection_similarity: null pointer");
  GB_REQUIRE(n1 > 0 && n2 > 0 && D > 0, "ghost_projection_similarity: empty dimension");
  GB_REQUIRE(ld1 >= D && ld2 >= D && ld_s >= n2, "ghost_projection_similarity: pitch smaller than the row it holds");
  const int bi = (n1 + 15) / 16, bj = (n2 + 15) / 16;
  GB_REQUIRE(bi <= 65535 && bj <= 65535, "ghost_projection_similarity: too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  GB_CUDA_OK(cudaMemset2DAsync(S, static_cast<size_t>(ld_s) * 4, 0, static_cast<size_t>(n2) * 4,
                               static_cast<size_t>(n1), st));
  SimParams p = {};
  p.P1 = P1; p.P2 = P2; p.n1 = n1; p.n2 = n2; p.D = D; p.ld1 = ld1; p.ld2 = ld2; p.scale = scale; p.S = S;
  p.ld_s = ld_s;
  // enough CTAs to fill the GPU a few times over, but no warp with fewer than 8 blocks of 16 elements
  const long long nkb = (D + 15) / 16;
  long long splits = (4ll * ds->sm_count + bi * bj - 1) / (static_cast<long long>(bi) * bj);
  const long long max_splits = (nkb + 63) / 64;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  const dim3 grid(static_cast<unsigned>(splits), static_cast<unsigned>(bi), static_cast<unsigned>(bj));
  const int esize = is_f32 ? 4 : 2;
  const bool vec = D % 4 == 0 && ld1 % 4 == 0 && ld2 % 4 == 0 &&
                   (reinterpret_cast<uintptr_t>(P1) % (4 * esize)) == 0 &&
                   (reinterpret_cast<uintptr_t>(P2) % (4 * esize)) == 0;
  if (is_f32) {
    if (vec) proj_similarity_kernel<float, true><<<grid, 256, 0, st>>>(p);
    else proj_similarity_kernel<float, false><<<grid, 256, 0, st>>>(p);
  } else {
    if (vec) proj_similarity_kernel<__nv_bfloat16, true><<<grid, 256, 0, st>>>(p);
    else proj_similarity_kernel<__nv_bfloat16, false><<<grid, 256, 0, st>>>(p);
  }
  count_launch();
  return post_launch("proj_similarity_kernel");
}
