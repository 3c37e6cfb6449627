// ghost_gram: the fused "ghost" dot-product kernel for Linear / Conv1D weights.
//
//   M[v, b] = sum_{t in sample b} sum_{s in sample v} (A_t . A_s) * (G_t . G_s)
//
// which is the Frobenius product of the per-sample weight gradients of train sample b and
// validation sample v (replaces the two GEMMs, the Hadamard product and the reductions of
// ghostEngines/supported_layers_grad_samplers_dotprod.py:119-130 and :416-437).  Train tokens are
// the M dimension, validation tokens the N dimension, and there are two contraction dimensions:
// d_in for the activation Gram and d_out for the output-gradient Gram.  Both 128 x BN Gram tiles
// are accumulated in tensor memory by tcgen05.mma, multiplied element-wise and reduced by the
// epilogue warps straight out of TMEM; the Gram matrices never exist in HBM.
//
// CTA layout (192 threads, persistent over tiles):
//   warps 0-3  epilogue: tcgen05.ld both accumulators, Hadamard, segmented reduce, atomicAdd to M
//   warp  4    TMA producer (one elected lane)
//   warp  5    TMEM allocator + MMA issuer (one elected lane)
// Pipeline: kStages shared-memory stages (train tile 128xBK + val tile BNxBK bf16 in 64-element atoms, 128B swizzle),
// full/empty mbarriers per stage, acc_full/acc_empty mbarriers per accumulator buffer.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace gb {

struct GramParams {
  long long rows_t;   // n_train * T
  long long rows_v;   // n_val * T
  long long T;
  int n_train, n_val;
  int ka, kg;         // contraction lengths (elements) of the activation / out-grad operands
  int m_tiles, n_tiles;
  int round_mode;     // 0: fp32 product of fp32 Grams; 1: round Grams and product to bf16
  float scale;
  float* M;           // [n_val, n_train]
  int* err;
};

template <int BN>
struct GramCfg {
  static constexpr int BM = 128;
  static constexpr int kAtomK = 64;                        // K elements of one 128-byte swizzle atom
  // K elements per stage.  BN = 128: two atoms per operand (64 KB stages), so the issuing thread
  // does one barrier round trip per eight MMAs; BN = 256 keeps one atom (48 KB stages), two would
  // leave room for two stages only.
  static constexpr int BK = (BN == 256) ? 64 : 128;
  static constexpr int kStageBytes = (BM + BN) * BK * 2;
  static constexpr int kStages = (BN == 256) ? 4 : 3;
  static constexpr int kAccBufs = 512 / (2 * BN);          // 1 (BN=256) or 2 (BN=128)
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN>
__global__ void __launch_bounds__(192, 1)
ghost_gram_kernel(const __grid_constant__ CUtensorMap tm_at, const __grid_constant__ CUtensorMap tm_av,
                  const __grid_constant__ CUtensorMap tm_gt, const __grid_constant__ CUtensorMap tm_gv,
                  const GramParams p) {
  using Cfg = GramCfg<BN>;
  constexpr int BM = Cfg::BM, BK = Cfg::BK, kStages = Cfg::kStages, kAccBufs = Cfg::kAccBufs;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
  uint64_t* full_bar = bars;                         // [kStages]
  uint64_t* empty_bar = bars + kStages;              // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;           // [kAccBufs]
  uint64_t* acc_empty = acc_full + kAccBufs;         // [kAccBufs]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kAccBufs);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.m_tiles * p.n_tiles;
  // Tiles are walked in bands of kBandM train tiles: inside a band the train index runs fastest, so
  // the ~148 tiles in flight at any time cover a near-square (train x val) patch and every operand
  // slice is fetched from HBM about once per patch and then shared through the L2.
  constexpr int kBandM = 16;
  auto tile_coords = [&](int tile, int& tm, int& tn) {
    const int band = tile / (kBandM * p.n_tiles);
    const int first = band * kBandM;
    const int rows = (p.m_tiles - first < kBandM) ? p.m_tiles - first : kBandM;
    const int local = tile - band * kBandM * p.n_tiles;
    tm = first + local % rows;
    tn = local / rows;
  };
  const int kb_a = (p.ka + BK - 1) / BK;
  const int kb_total = kb_a + (p.kg + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < kAccBufs; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_at);
    tma_prefetch_desc(&tm_av);
    tma_prefetch_desc(&tm_gt);
    tma_prefetch_desc(&tm_gv);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tm, tn);
        const int m0 = tm * BM;
        const int n0 = tn * BN;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, 401)) { ok = false; break; }
          uint8_t* st = smem + stage * Cfg::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          // stage layout: train atoms, then validation atoms; an atom past the end of K is
          // zero-filled by the bounds check
          const CUtensorMap* mt = (kb < kb_a) ? &tm_at : &tm_gt;
          const CUtensorMap* mv = (kb < kb_a) ? &tm_av : &tm_gv;
          const int k0 = ((kb < kb_a) ? kb : kb - kb_a) * BK;
#pragma unroll
          for (int a = 0; a < BK / Cfg::kAtomK; ++a) {
            tma_load_2d(st + a * (BM * Cfg::kAtomK * 2), mt, &full_bar[stage], k0 + a * Cfg::kAtomK, m0);
            tma_load_2d(st + BM * BK * 2 + a * (BN * Cfg::kAtomK * 2), mv, &full_bar[stage],
                        k0 + a * Cfg::kAtomK, n0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.err, 502)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_a = tmem_base + acc * (2 * BN);
        const uint32_t d_g = d_a + BN;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.err, 503)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const bool first = (kb == 0) || (kb == kb_a);
          const uint32_t dst = (kb < kb_a) ? d_a : d_g;
#pragma unroll
          for (int a = 0; a < BK / Cfg::kAtomK; ++a) {
            const uint64_t adesc = make_smem_desc_sw128(sa + a * (BM * Cfg::kAtomK * 2), 16, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(sa + BM * BK * 2 + a * (BN * Cfg::kAtomK * 2), 16, 1024);
#pragma unroll
            for (int k = 0; k < Cfg::kAtomK / 16; ++k)
              umma_bf16(dst, adesc + 2 * k, bdesc + 2 * k, idesc, (first && a == 0 && k == 0) ? 0u : 1u);
          }
          umma_commit(&empty_bar[stage]);   // frees the stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&acc_full[acc]);
        if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-3)
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, tm, tn);
      const long long m0 = static_cast<long long>(tm) * BM;
      const long long n0 = static_cast<long long>(tn) * BN;
      if (!mbar_wait_warp(&acc_full[acc], acc_phase, abort_flag, p.err, 104)) break;
      tc_fence_after_sync();

      const long long row = m0 + threadIdx.x;
      const bool row_ok = row < p.rows_t;
      const int b = row_ok ? static_cast<int>(row / p.T) : -1;
      // rows are ascending, so the warp covers one train sample iff its first and last rows agree
      const int b_first = __shfl_sync(0xffffffffu, b, 0);
      const int b_last = __shfl_sync(0xffffffffu, b, 31);
      const bool warp_uniform = (b_first == b_last) && (b_first >= 0);

      int cur_v = static_cast<int>(n0 / p.T);
      long long boundary = static_cast<long long>(cur_v + 1) * p.T - n0;   // tile-relative column
      float sum = 0.f;
      const uint32_t t_a = tmem_base + lane_base + acc * (2 * BN);
      const uint32_t t_g = t_a + BN;

      auto flush = [&](float val, int v) {
        if (v >= p.n_val) return;
        val *= p.scale;
        if (warp_uniform) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) val += __shfl_xor_sync(0xffffffffu, val, o);
          if (lane == 0) atomicAdd(&p.M[static_cast<long long>(v) * p.n_train + b_first], val);
        } else if (row_ok) {
          atomicAdd(&p.M[static_cast<long long>(v) * p.n_train + b], val);
        }
      };

#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t ra[32], rg[32];
        tmem_ld32(t_a + c0, ra);
        tmem_ld32(t_g + c0, rg);
        tmem_ld_wait();
        if (c0 + 32 <= boundary) {
          if (p.round_mode == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) sum = fmaf(__uint_as_float(ra[j]), __uint_as_float(rg[j]), sum);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              sum += bf16_round(bf16_round(__uint_as_float(ra[j])) * bf16_round(__uint_as_float(rg[j])));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j == boundary) {
              flush(sum, cur_v);
              sum = 0.f;
              ++cur_v;
              boundary += p.T;
            }
            const float x = __uint_as_float(ra[j]), y = __uint_as_float(rg[j]);
            sum += (p.round_mode == 0) ? x * y : bf16_round(bf16_round(x) * bf16_round(y));
          }
        }
      }
      // every TMEM read of this tile is done: hand the accumulator back before the atomics
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      flush(sum, cur_v);
      if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int BN>
static int launch_gram(const void* a_t, const void* a_v, const void* g_t, const void* g_v,
                       int n_train, int n_val, long long T, int ka, int kg, long long ld_at,
                       long long ld_av, long long ld_gt, long long ld_gv, int round_mode, float scale,
                       float* M, const DeviceState* ds, cudaStream_t stream) {
  using Cfg = GramCfg<BN>;
  GramParams p;
  p.rows_t = static_cast<long long>(n_train) * T;
  p.rows_v = static_cast<long long>(n_val) * T;
  p.T = T;
  p.n_train = n_train;
  p.n_val = n_val;
  p.ka = ka;
  p.kg = kg;
  p.m_tiles = ceil_div(p.rows_t, Cfg::BM);
  p.n_tiles = ceil_div(p.rows_v, BN);
  p.round_mode = round_mode;
  p.scale = scale;
  p.M = M;
  p.err = ds->err_word;
  CUtensorMap tm_at, tm_av, tm_gt, tm_gv;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tm_at, a_t, p.rows_t, ka, ld_at, Cfg::BM)) != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_2d(&tm_av, a_v, p.rows_v, ka, ld_av, BN)) != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_2d(&tm_gt, g_t, p.rows_t, kg, ld_gt, Cfg::BM)) != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_2d(&tm_gv, g_v, p.rows_v, kg, ld_gv, BN)) != GHOST_OK) return rc;

  static bool attr_set[64] = {};
  if (!attr_set[ds->device]) {
    GB_CUDA_OK(cudaFuncSetAttribute(ghost_gram_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kSmemBytes));
    attr_set[ds->device] = true;
  }
  const long long tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
  const int grid = static_cast<int>(tiles < ds->sm_count ? tiles : ds->sm_count);
  ghost_gram_kernel<BN><<<grid, 192, Cfg::kSmemBytes, stream>>>(tm_at, tm_av, tm_gt, tm_gv, p);
  count_launch();
  return post_launch("ghost_gram_kernel");
}

int launch_gram_pair(const void* a_t, const void* a_v, const void* g_t, const void* g_v, int n_train, int n_val,
                     long long T, int ka, int kg, long long ld_at, long long ld_av, long long ld_gt,
                     long long ld_gv, int round_mode, float scale, float* M, const DeviceState* ds,
                     cudaStream_t stream);

// 0: single-CTA kernels only; 1: CTA-pair kernel for problems with at least 512 train tokens and 256
// to 8192 validation tokens (where it measured faster: 1474 against 1339 TFLOP/s with 32768 x 4096
// tokens, 985 against 1117 with 131072 x 16384); 2: CTA-pair kernel from 512 x 256 tokens up
static int g_gram_pair_mode = 1;
bool xty_pair_usable(const DeviceState* ds);     // a cluster of two ~198 KB CTAs fits on the device

}  // namespace gb

extern "C" int ghost_set_gram_pair_mode(int mode) {
  if (mode < 0 || mode > 2) return GHOST_ERR_INVALID;
  gb::g_gram_pair_mode = mode;
  return GHOST_OK;
}

extern "C" int ghost_gram_dot_bf16(const void* a_train, const void* a_val, const void* g_train,
                                   const void* g_val, int n_train, int n_val, long long T, int ka,
                                   int kg, long long ld_at, long long ld_av, long long ld_gt,
                                   long long ld_gv, int round_mode, float scale, float* M_out,
                                   void* stream) {
  using namespace gb;
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(a_train && a_val && g_train && g_val && M_out, "ghost_gram_dot_bf16: null pointer");
  GB_REQUIRE(n_train > 0, "No training samples to compute dot product, check batch sizes.");
  GB_REQUIRE(n_val > 0 && T > 0 && ka > 0 && kg > 0, "ghost_gram_dot_bf16: empty dimension");
  GB_REQUIRE(round_mode == 0 || round_mode == 1, "ghost_gram_dot_bf16: round_mode must be 0 or 1");
  GB_REQUIRE(static_cast<long long>(n_train) * T < (1ll << 31) - 256 &&
             static_cast<long long>(n_val) * T < (1ll << 31) - 256,
             "ghost_gram_dot_bf16: more than 2^31 tokens");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  GB_CUDA_OK(cudaMemsetAsync(M_out, 0, sizeof(float) * static_cast<size_t>(n_val) * n_train, st));
  const long long rows_v = static_cast<long long>(n_val) * T;
  const bool pair_wanted = g_gram_pair_mode == 2 || (g_gram_pair_mode == 1 && rows_v <= 8192);
  if (pair_wanted && rows_v >= 256 && static_cast<long long>(n_train) * T >= 512 && xty_pair_usable(ds))
    return launch_gram_pair(a_train, a_val, g_train, g_val, n_train, n_val, T, ka, kg, ld_at, ld_av, ld_gt,
                            ld_gv, round_mode, scale, M_out, ds, st);
  if (rows_v <= 128)
    return launch_gram<128>(a_train, a_val, g_train, g_val, n_train, n_val, T, ka, kg, ld_at, ld_av,
                            ld_gt, ld_gv, round_mode, scale, M_out, ds, st);
  return launch_gram<256>(a_train, a_val, g_train, g_val, n_train, n_val, T, ka, kg, ld_at, ld_av,
                          ld_gt, ld_gv, round_mode, scale, M_out, ds, st);
}
