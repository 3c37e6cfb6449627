// gradproj_fused: per-sample Kronecker-projected weight gradients
//
//   out[b] = scale * (G_b P_r^T)^T (A_b P_c^T)            [k_r, k_c] fp32 per sample
//
// (ghostEngines/gradProjection/autograd_gradproj.py:120-165: for nn.Linear P_r = P_o, P_c = P_i and
// the result is [k_o, k_i]; for HF Conv1D the reference swaps the roles, P_r = P_i, P_c = P_o, and
// the result is [k_i, k_o].)  The activations and output gradients are streamed from HBM exactly
// once: per 128-token chunk the two skinny projections run on tcgen05 (TMA-fed, accumulators in
// TMEM), the projected [128, k] blocks are moved TMEM -> shared memory as fp32, and the small
// k_r x k_c contraction over the chunk's tokens is done in registers by the epilogue warps
// (< 1 % of the flops).  Results go straight into the caller's [B, total_proj_dim] row slices with
// fp32 atomics, so no [B, T, k] intermediate ever reaches HBM.  HBM-bound by design: arithmetic
// intensity is about k flop per byte.  What has to be kept small is the per-stage cost of the two
// single threads that drive the pipeline (a barrier wait, an expect-tx, the TMA and MMA issues --
// each on the order of 100 cycles), hence wide stages and one multi-lane TMA instruction per stage.
//
// CTA layout (192 threads): warps 0-3 epilogue, warp 4 TMA producer, warp 5 MMA issuer.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace gb {

struct GpParams {
  int B;
  long long T;
  int n_r, n_c;            // contraction lengths: columns of G / of A (already padded & stacked)
  int k_r, k_c;            // projection ranks (rows of P_r / P_c)
  int kr_pad, kc_pad;      // MMA N extents (multiples of 16)
  int chunks_per_sample;
  long long units;         // B * chunks_per_sample
  int units_per_cta;       // base number of units per CTA
  int units_extra;         // the first `units_extra` CTAs take one more
  float scale;
  float* out;              // sample b at out + b * out_stride, [k_r, k_c] row-major
  long long out_stride;
  int* err;
};

template <int KMAX>   // largest padded rank this instantiation handles (32, 64 or 128)
struct GpCfg {
  static constexpr int BM = 128, BK = 64;                  // BK: one 128-byte swizzle atom of bf16
  // Columns per pipeline stage = ATOMS * 64.  The single threads that drive the pipeline pay a few
  // hundred cycles per stage for the barrier round trip, so a stage carries two atoms when the
  // shared memory allows it.
  static constexpr int ATOMS = (KMAX == 128) ? 1 : 2;
  static constexpr int kActAtomBytes = BM * BK * 2;
  static constexpr int kProjAtomBytes = KMAX * BK * 2;
  static constexpr int kStageBytes = ATOMS * (kActAtomBytes + kProjAtomBytes);
  // The pipeline is bound by how many bytes are in flight per SM, so the fp32 staging of the
  // projected blocks is kept to half a tile (64 tokens at a time) and the rest goes to stages.
  static constexpr int kStageRows = 64;
  static constexpr int kProjBytes = 2 * kStageRows * KMAX * 4;
  static constexpr int kStages = (KMAX == 32) ? 5 : (KMAX == 64 ? 4 : 5);     // fills the 227 KB of shared memory
  static constexpr int kSmemBytes = kStages * kStageBytes + kProjBytes + 1024 + 256;
  static constexpr int RT = KMAX / 16;   // output rows per thread (16 thread rows)
  static constexpr int CT = KMAX / 8;    // output cols per thread (8 thread cols)
  static constexpr int NCH = KMAX / 4;   // float4 chunks per staged row
};

// Staged fp32 rows are stored with their float4 chunks XOR-permuted by the row index, so that the
// 32 lanes of a warp (32 consecutive rows, same chunk) spread over all banks.
template <int KMAX>
__device__ __forceinline__ int gp_staged_index(int row, int elem) {
  return row * KMAX + ((((elem >> 2) ^ row) & (KMAX / 4 - 1)) << 2) + (elem & 3);
}

template <int KMAX>
__global__ void __launch_bounds__(192, 1)
gradproj_kernel(const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ CUtensorMap tm_pr,
                const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_pc,
                const GpParams p) {
  using Cfg = GpCfg<KMAX>;
  constexpr int BM = Cfg::BM, BK = Cfg::BK, kStages = Cfg::kStages, RT = Cfg::RT, CT = Cfg::CT;
  constexpr int ATOMS = Cfg::ATOMS;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_r = reinterpret_cast<float*>(smem + kStages * Cfg::kStageBytes);   // [64][KMAX]
  float* s_c = s_r + Cfg::kStageRows * KMAX;                                  // [64][KMAX]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes + Cfg::kProjBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* acc_full = bars + 2 * kStages;    // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long bx = blockIdx.x;
  const long long u0 = bx * p.units_per_cta + (bx < p.units_extra ? bx : p.units_extra);
  long long u1 = u0 + p.units_per_cta + (bx < p.units_extra ? 1 : 0);
  if (u1 > p.units) u1 = p.units;
  const int kb_r = (p.n_r + ATOMS * BK - 1) / (ATOMS * BK);            // pipeline stages over G's columns
  const int kb_total = kb_r + (p.n_c + ATOMS * BK - 1) / (ATOMS * BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_g); tma_prefetch_desc(&tm_pr); tma_prefetch_desc(&tm_a); tma_prefetch_desc(&tm_pc);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // Producer warp.  Lane 0 owns the barriers; lanes [0, ATOMS) each issue the TMA of one
    // activation atom and lanes [ATOMS, 2*ATOMS) the TMA of one projection atom -- one warp
    // instruction per stage instead of one thread issuing the boxes back to back.
    const bool is_p = lane >= ATOMS;
    const int atom = is_p ? lane - ATOMS : lane;
    const uint32_t dst_off = is_p ? ATOMS * Cfg::kActAtomBytes + atom * Cfg::kProjAtomBytes
                                  : atom * Cfg::kActAtomBytes;
    int stage = 0; uint32_t phase = 0; bool ok = true;
    for (long long u = u0; u < u1 && ok; ++u) {
      const int b = static_cast<int>(u / p.chunks_per_sample);
      const int row0 = static_cast<int>(u % p.chunks_per_sample) * BM;
      for (int kb = 0; kb < kb_total; ++kb) {
        int w = 1;
        if (lane == 0) w = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, 421) ? 1 : 0;
        w = __shfl_sync(0xffffffffu, w, 0);
        if (!w) { ok = false; break; }
        const bool first = kb < kb_r;
        if (lane == 0)
          mbar_arrive_expect_tx(&full_bar[stage], ATOMS * (BM + (first ? p.kr_pad : p.kc_pad)) * BK * 2);
        if (lane < 2 * ATOMS) {
          // an atom past the last column starts out of range and is zero-filled
          const int col = ((first ? kb : kb - kb_r) * ATOMS + atom) * BK;
          const CUtensorMap* m = first ? (is_p ? &tm_pr : &tm_g) : (is_p ? &tm_pc : &tm_a);
          tma_load_3d(smem + stage * Cfg::kStageBytes + dst_off, m, &full_bar[stage], col,
                      is_p ? 0 : row0, is_p ? 0 : b);
        }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc_r = make_idesc_bf16(BM, p.kr_pad, 0, 0);
      const uint32_t idesc_c = make_idesc_bf16(BM, p.kc_pad, 0, 0);
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      for (long long u = u0; u < u1 && ok; ++u) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.err, 522)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_r = tmem_base + acc * 256;
        const uint32_t d_c = d_r + 128;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.err, 523)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const bool first = kb < kb_r;
          const bool fresh = (kb == 0) || (kb == kb_r);
          const uint32_t d = first ? d_r : d_c;
          const uint32_t idesc = first ? idesc_r : idesc_c;
#pragma unroll
          for (int at = 0; at < ATOMS; ++at) {
            const uint64_t adesc = make_smem_desc_sw128(sa + at * Cfg::kActAtomBytes, 16, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(sa + ATOMS * Cfg::kActAtomBytes + at * Cfg::kProjAtomBytes, 16, 1024);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_bf16(d, adesc + 2 * k, bdesc + 2 * k, idesc, (fresh && at == 0 && k == 0) ? 0u : 1u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: warps 0-3
    const int tid = threadIdx.x;              // 0..127 = token row inside the chunk
    const int ty = tid >> 3, tx = tid & 7;    // 16 x 8 thread grid over the [k_r, k_c] output
    float o[RT][CT];
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
      for (int j = 0; j < CT; ++j) o[i][j] = 0.f;
    int cur_b = -1;
    int acc = 0; uint32_t acc_phase = 0;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;

    auto flush = [&](int b) {
      float* dst = p.out + static_cast<long long>(b) * p.out_stride;
#pragma unroll
      for (int i = 0; i < RT; ++i) {
        const int r = ty * RT + i;
#pragma unroll
        for (int j = 0; j < CT; ++j) {
          const int c = tx * CT + j;
          if (r < p.k_r && c < p.k_c && o[i][j] != 0.f)
            atomicAdd(dst + static_cast<long long>(r) * p.k_c + c, o[i][j] * p.scale);
          o[i][j] = 0.f;
        }
      }
    };
    // TMEM -> shared (fp32): row `tid` of one projected block
    auto stage_block = [&](uint32_t taddr, int kpad, float* dst) {
#pragma unroll 1
      for (int c0 = 0; c0 < kpad; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          if (c0 + j < KMAX)
            *reinterpret_cast<float4*>(&dst[gp_staged_index<KMAX>(tid & 63, c0 + j)]) =
                make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      }
    };

    bool alive = true;
    for (long long u = u0; u < u1; ++u) {
      const int b = static_cast<int>(u / p.chunks_per_sample);
      if (b != cur_b) { if (cur_b >= 0) flush(cur_b); cur_b = b; }
      if (!named_bar_and(2, 128, mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.err, 124))) { alive = false; break; }
      tc_fence_after_sync();
      const uint32_t t_r = tmem_base + lane_base + acc * 256;
      // two halves of 64 tokens: warps 0-1 own TMEM lanes 0-63, warps 2-3 lanes 64-127
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        if ((warp >> 1) == half) {
          stage_block(t_r, p.kr_pad, s_r);
          stage_block(t_r + 128, p.kc_pad, s_c);
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[acc]);     // four arrivals per tile, one per warp
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");     // the four epilogue warps only
        // out[r, c] += sum_t s_r[t][r] * s_c[t][c]
#pragma unroll 4
        for (int t = 0; t < Cfg::kStageRows; ++t) {
          float rr[RT], cc[CT];
          if constexpr (RT >= 4) {
#pragma unroll
            for (int i = 0; i < RT; i += 4)
              *reinterpret_cast<float4*>(&rr[i]) = *reinterpret_cast<const float4*>(&s_r[gp_staged_index<KMAX>(t, ty * RT + i)]);
          } else {
            *reinterpret_cast<float2*>(&rr[0]) = *reinterpret_cast<const float2*>(&s_r[gp_staged_index<KMAX>(t, ty * RT)]);
          }
#pragma unroll
          for (int j = 0; j < CT; j += 4)
            *reinterpret_cast<float4*>(&cc[j]) = *reinterpret_cast<const float4*>(&s_c[gp_staged_index<KMAX>(t, tx * CT + j)]);
#pragma unroll
          for (int i = 0; i < RT; ++i)
#pragma unroll
            for (int j = 0; j < CT; ++j) o[i][j] = fmaf(rr[i], cc[j], o[i][j]);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (alive && cur_b >= 0) flush(cur_b);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) { tc_fence_after_sync(); tmem_dealloc(tmem_base, 512); }
}

template <int KMAX>
static int launch_gradproj(const CUtensorMap& tg, const CUtensorMap& tpr, const CUtensorMap& ta,
                           const CUtensorMap& tpc, GpParams& p, const DeviceState* ds, cudaStream_t st) {
  using Cfg = GpCfg<KMAX>;
  static bool attr_set[64] = {};
  if (!attr_set[ds->device]) {
    GB_CUDA_OK(cudaFuncSetAttribute(gradproj_kernel<KMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set[ds->device] = true;
  }
  const int grid = static_cast<int>(p.units < ds->sm_count ? p.units : ds->sm_count);
  p.units_per_cta = static_cast<int>(p.units / grid);
  p.units_extra = static_cast<int>(p.units % grid);
  gradproj_kernel<KMAX><<<grid, 192, Cfg::kSmemBytes, st>>>(tg, tpr, ta, tpc, p);
  count_launch();
  return post_launch("gradproj_kernel");
}

}  // namespace gb

using namespace gb;

// G: [B, T, n_r] bf16 (pitch ldg), A: [B, T, n_c] bf16 (pitch lda), P_r: [k_r, n_r] bf16 (pitch ldpr),
// P_c: [k_c, n_c] bf16 (pitch ldpc).  out + b * out_stride receives [k_r, k_c] fp32 (overwritten).
extern "C" int ghost_gradproj_dense_bf16(const void* G, const void* A, int B, long long T, int n_r, int n_c,
                                         long long ldg, long long lda, const void* P_r, const void* P_c,
                                         int k_r, int k_c, long long ldpr, long long ldpc, float scale,
                                         float* out, long long out_stride, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(G && A && P_r && P_c && out, "ghost_gradproj_dense_bf16: null pointer");
  GB_REQUIRE(B > 0 && T > 0 && n_r > 0 && n_c > 0 && k_r > 0 && k_c > 0, "ghost_gradproj_dense_bf16: empty dimension");
  GB_REQUIRE(k_r <= 128 && k_c <= 128, "ghost_gradproj_dense_bf16: projection ranks above 128 are not supported");
  GB_REQUIRE(out_stride >= static_cast<long long>(k_r) * k_c, "ghost_gradproj_dense_bf16: out_stride smaller than k_r * k_c");
  GB_REQUIRE(T < (1ll << 31) - 128, "ghost_gradproj_dense_bf16: T too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  GpParams p = {};
  p.B = B; p.T = T; p.n_r = n_r; p.n_c = n_c; p.k_r = k_r; p.k_c = k_c;
  p.kr_pad = (k_r + 15) / 16 * 16;
  p.kc_pad = (k_c + 15) / 16 * 16;
  p.chunks_per_sample = ceil_div(T, 128);
  p.units = static_cast<long long>(B) * p.chunks_per_sample;
  p.scale = scale;
  p.out = out;
  p.out_stride = out_stride;
  p.err = ds->err_word;
  CUtensorMap tg, tpr, ta, tpc;
  int rc;
  if ((rc = make_tmap_bf16_3d(&tg, G, B, T, n_r, ldg, 128)) != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_3d(&ta, A, B, T, n_c, lda, 128)) != GHOST_OK) return rc;
  // the projection matrices as one-sample 3-D operands, so that one TMA instruction form serves all four
  if ((rc = make_tmap_bf16_3d(&tpr, P_r, 1, k_r, n_r, ldpr, p.kr_pad)) != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_3d(&tpc, P_c, 1, k_c, n_c, ldpc, p.kc_pad)) != GHOST_OK) return rc;
  GB_CUDA_OK(cudaMemset2DAsync(out, out_stride * sizeof(float), 0, static_cast<size_t>(k_r) * k_c * sizeof(float), B, st));
  const int kmax = p.kr_pad > p.kc_pad ? p.kr_pad : p.kc_pad;
  if (kmax <= 32) return launch_gradproj<32>(tg, tpr, ta, tpc, p, ds, st);
  if (kmax <= 64) return launch_gradproj<64>(tg, tpr, ta, tpc, p, ds, st);
  return launch_gradproj<128>(tg, tpr, ta, tpc, p, ds, st);
}
