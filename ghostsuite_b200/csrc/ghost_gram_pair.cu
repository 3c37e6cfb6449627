// ghost_gram, CTA-pair variant (tcgen05 cta_group::2).  Same math and epilogue as ghost_gram.cu:
//   M[v, b] = sum_{t in b, s in v} (A_t . A_s)(G_t . G_s)
// A cluster of two CTAs owns a 256 (train tokens) x 256 (validation tokens) tile.  CTA r loads its
// own 128 train rows and its own 128 of the 256 validation rows (64 KB per stage of 128 K-elements,
// three stages: eight MMAs per barrier round trip of the issuing thread), the leader CTA issues
// 256x256x16 MMAs that read both CTAs' shared memory, and each CTA
// reduces its own 128 accumulator rows out of its own tensor memory.  Per output element the
// validation operand crosses L2 -> shared memory half as often as in the single-CTA kernel.
//
// Barriers: full[s] lives in the leader and collects the bytes of both CTAs' loads; empty[s] and
// acc_full exist in both CTAs and are signalled by the leader's tcgen05.commit to the pair;
// acc_empty lives in the leader and counts the eight epilogue warps of the pair.  All mbarrier
// waits are bounded; the cluster barrier before teardown is reached by every thread.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace gb {

struct GramPairParams {
  long long rows_t, rows_v, T;
  int n_train, n_val;
  int ka, kg;
  int m_tiles, n_tiles;     // 256 x 256 tiles
  int round_mode;
  float scale;
  float* M;
  int* err;
};

struct GramPairCfg {
  static constexpr int BM = 128;           // rows per CTA
  static constexpr int BNH = 128;          // validation rows loaded per CTA (half of N = 256)
  static constexpr int BN = 256;
  static constexpr int BK = 128;           // K elements per stage = two 64-element swizzle atoms per operand
  static constexpr int kAtomK = 64;
  static constexpr int kStageBytes = (BM + BNH) * BK * 2;   // 64 KB
  static constexpr int kStages = 3;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
ghost_gram_pair_kernel(const __grid_constant__ CUtensorMap tm_at, const __grid_constant__ CUtensorMap tm_av,
                       const __grid_constant__ CUtensorMap tm_gt, const __grid_constant__ CUtensorMap tm_gv,
                       const GramPairParams p) {
  using Cfg = GramPairCfg;
  constexpr int BM = Cfg::BM, BNH = Cfg::BNH, BN = Cfg::BN, BK = Cfg::BK, kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
  uint64_t* full_bar = bars;                 // used in the leader only
  uint64_t* empty_bar = bars + kStages;      // both CTAs
  uint64_t* acc_full = bars + 2 * kStages;   // both CTAs
  uint64_t* acc_empty = acc_full + 1;        // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = p.m_tiles * p.n_tiles;
  constexpr int kBandM = 8;
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
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);      // 4 epilogue warps in each CTA of the pair
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_at);
    tma_prefetch_desc(&tm_av);
    tma_prefetch_desc(&tm_gt);
    tma_prefetch_desc(&tm_gv);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers are initialised before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        tile_coords(tile, tm, tn);
        const int m0 = tm * (2 * BM) + static_cast<int>(rank) * BM;
        const int n0 = tn * BN + static_cast<int>(rank) * BNH;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, 441)) { ok = false; break; }
          uint8_t* st = smem + stage * Cfg::kStageBytes;
          // the leader's barrier collects both CTAs' bytes
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          // stage layout: [train atom 0 | train atom 1 | validation atom 0 | validation atom 1]; an atom
          // past the end of K is zero-filled by the bounds check
          const CUtensorMap* mt = (kb < kb_a) ? &tm_at : &tm_gt;
          const CUtensorMap* mv = (kb < kb_a) ? &tm_av : &tm_gv;
          const int k0 = ((kb < kb_a) ? kb : kb - kb_a) * BK;
#pragma unroll
          for (int a = 0; a < BK / Cfg::kAtomK; ++a) {
            tma_load_2d_pair(st + a * (BM * Cfg::kAtomK * 2), mt, bar, k0 + a * Cfg::kAtomK, m0);
            tma_load_2d_pair(st + BM * BK * 2 + a * (BNH * Cfg::kAtomK * 2), mv, bar, k0 + a * Cfg::kAtomK, n0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait(acc_empty, acc_phase ^ 1, abort_flag, p.err, 542)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_a = tmem_base;
        const uint32_t d_g = tmem_base + BN;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.err, 543)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const bool first = (kb == 0) || (kb == kb_a);
          const uint32_t dst = (kb < kb_a) ? d_a : d_g;
#pragma unroll
          for (int a = 0; a < BK / Cfg::kAtomK; ++a) {
            const uint64_t adesc = make_smem_desc_sw128(sa + a * (BM * Cfg::kAtomK * 2), 16, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(sa + BM * BK * 2 + a * (BNH * Cfg::kAtomK * 2), 16, 1024);
#pragma unroll
            for (int k = 0; k < Cfg::kAtomK / 16; ++k)
              umma_bf16_pair(dst, adesc + 2 * k, bdesc + 2 * k, idesc, (first && a == 0 && k == 0) ? 0u : 1u);
          }
          umma_commit_pair(&empty_bar[stage], 3);      // frees the stage in both CTAs
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(acc_full, 3);
        acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-3, both CTAs)
    uint32_t acc_phase = 0;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t acc_empty_leader = map_to_cta(smem_u32(acc_empty), 0);
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      int tm, tn;
      tile_coords(tile, tm, tn);
      const long long m0 = static_cast<long long>(tm) * (2 * BM) + static_cast<long long>(rank) * BM;
      const long long n0 = static_cast<long long>(tn) * BN;
      if (!mbar_wait_warp(acc_full, acc_phase, abort_flag, p.err, 144)) break;
      tc_fence_after_sync();

      const long long row = m0 + threadIdx.x;
      const bool row_ok = row < p.rows_t;
      const int b = row_ok ? static_cast<int>(row / p.T) : -1;
      const int b_first = __shfl_sync(0xffffffffu, b, 0);
      const int b_last = __shfl_sync(0xffffffffu, b, 31);
      const bool warp_uniform = (b_first == b_last) && (b_first >= 0);

      int cur_v = static_cast<int>(n0 / p.T);
      long long boundary = static_cast<long long>(cur_v + 1) * p.T - n0;
      float sum = 0.f;
      const uint32_t t_a = tmem_base + lane_base;
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
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
      flush(sum, cur_v);
      acc_phase ^= 1;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();          // no CTA leaves while its peer may still signal or read it
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

int launch_gram_pair(const void* a_t, const void* a_v, const void* g_t, const void* g_v, int n_train, int n_val,
                     long long T, int ka, int kg, long long ld_at, long long ld_av, long long ld_gt,
                     long long ld_gv, int round_mode, float scale, float* M, const DeviceState* ds,
                     cudaStream_t stream) {
  using Cfg = GramPairCfg;
  GramPairParams p;
  p.rows_t = static_cast<long long>(n_train) * T;
  p.rows_v = static_cast<long long>(n_val) * T;
  p.T = T;
  p.n_train = n_train;
  p.n_val = n_val;
  p.ka = ka;
  p.kg = kg;
  p.m_tiles = ceil_div(p.rows_t, 2 * Cfg::BM);
  p.n_tiles = ceil_div(p.rows_v, Cfg::BN);
  p.round_mode = round_mode;
  p.scale = scale;
  p.M = M;
  p.err = ds->err_word;
  CUtensorMap tm_at, tm_av, tm_gt, tm_gv;
  int rc;
  if ((rc = make_tmap_bf16_2d(&tm_at, a_t, p.rows_t, ka, ld_at, Cfg::BM)) != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_2d(&tm_av, a_v, p.rows_v, ka, ld_av, Cfg::BNH)) != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_2d(&tm_gt, g_t, p.rows_t, kg, ld_gt, Cfg::BM)) != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_2d(&tm_gv, g_v, p.rows_v, kg, ld_gv, Cfg::BNH)) != GHOST_OK) return rc;
  static bool attr_set[64] = {};
  if (!attr_set[ds->device]) {
    GB_CUDA_OK(cudaFuncSetAttribute(ghost_gram_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kSmemBytes));
    attr_set[ds->device] = true;
  }
  const long long tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
  long long pairs = ds->sm_count / 2;
  if (pairs > tiles) pairs = tiles;
  ghost_gram_pair_kernel<<<static_cast<int>(2 * pairs), 192, Cfg::kSmemBytes, stream>>>(tm_at, tm_av, tm_gt, tm_gv, p);
  count_launch();
  return post_launch("ghost_gram_pair_kernel");
}

}  // namespace gb
