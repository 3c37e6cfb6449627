// xty_gemm, CTA-pair variant (tcgen05 cta_group::2) of the per-sample tile pass and of the
// train-gradient (split-K) pass.
//
// Tile pass: same math and the same stored layout as xty_gemm.cu's tile-store mode: for every sample s and
// every 128 x 256 tile, D = X_s[:, m-block]^T Y_s[:, n-block] contracted over the sample's tokens,
// written tile-major ([tile][sample][128][256], bf16 or fp32).  A cluster of two CTAs owns a 256 x 256
// block of the per-sample gradient: CTA r loads its own 128 X columns and its own 128 of the 256 Y
// columns (64 KB per stage of 128 tokens, three stages), the leader issues 256 x 256 x 16 MMAs that
// read both CTAs' shared memory (eight per stage: with 64-token stages the issuing thread spent as
// long on the two barrier operations of a stage as the tensor core on its four MMAs), and each CTA writes the 128 x 256 tile that
// sits in its own tensor memory: bf16 tiles through two swizzled [128][32] staging boxes in shared
// memory that the copy engine stores (cp.async.bulk.tensor, shared -> global), fp32 tiles with
// 256-bit stores.  Per output element the Y operand crosses L2 -> shared memory and
// shared memory -> tensor core half as often as in the single-CTA kernel.
//
// Train-gradient pass (one "sample" holding all token rows): a unit is a 256 x 256 block and one of
// k_splits ranges of 128-row blocks; units are walked split-major, so the pairs running at the same
// time read the same token rows; every CTA adds its 128 x 256 half into the fp32 workspace with
// red.global.add.v4.f32, exactly as the single-CTA kernel does.
//
// Barriers: full[s] lives in the leader and collects the bytes of both CTAs' loads; empty[s] and
// acc_full[a] exist in both CTAs and are signalled by the leader's tcgen05.commit to the pair;
// acc_empty[a] lives in the leader and counts the eight epilogue warps of the pair.  All mbarrier
// waits are bounded; the cluster barrier before teardown is reached by every thread.  Every CTA
// fetches what it needs itself.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "xty_colsum.cuh"

namespace gb {

struct XtyPairParams {
  int m_cols, n_cols;
  int m_tiles128;            // 128-row tiles of the stored layout (X columns)
  int m_tiles, n_tiles;      // 256 x 256 blocks
  int samples, sample0;
  long long T;
  void* vgrad;
  int v_is_f32;
  int tma_store;             // bf16 tiles: staged in shared memory and stored by the copy engine
  int accumulate;            // 0: store tiles; 1: add into acc_ws ("samples" = k_splits, one real sample)
  int kb_per_split;          // row blocks (BK tokens) per split (accumulate)
  float* acc_ws;             // [m_cols, ld_acc] fp32, zeroed by the host
  long long ld_acc;
  // per-sample column sums of one operand (the bias terms' input), taken by four extra warps that
  // read the operand rows through L2 while the tensor core works: 0 none, 1 X, 2 Y
  int cs_of;
  const __nv_bfloat16* cs_src;   // that operand, [n_samples_total, T, cs_cols], row pitch cs_ld
  long long cs_ld;
  int cs_cols;
  float* cs_out;             // [n_samples_total, cs_cols] fp32
  int* err;
};

struct XtyPairCfg {
  static constexpr int BM = 128;           // X columns per CTA
  static constexpr int BNH = 128;          // Y columns loaded per CTA (half of N = 256)
  static constexpr int BN = 256;
  static constexpr int BK = 128;           // tokens per stage: eight MMAs per barrier round trip
  static constexpr int kStageBytes = (BM + BNH) * BK * 2;   // 64 KB
  static constexpr int kStages = 3;
  static constexpr int kColsumBytes = 8 * 128 * 4;          // cross-row-lane reduction of the column-sum warps
  // bf16 tiles leave through shared memory: two [128 rows][32 columns] boxes (64-byte rows, 64-byte
  // swizzle) that the epilogue warps fill alternately and one thread hands to the copy engine
  static constexpr int kStoreBoxBytes = 128 * 32 * 2;
  static constexpr int kStoreBytes = 2 * kStoreBoxBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 256 + kColsumBytes;
};

__device__ __forceinline__ void st_global_v8_pair(void* addr, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(addr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
// 32 consecutive accumulator columns of one output row -> fp32 workspace (16-byte aligned rows)
__device__ __forceinline__ void red_add_row32_pair(float* dst, const uint32_t (&r)[32], int ncol) {
  if (ncol >= 32) {
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "f"(__uint_as_float(r[j])),
                   "f"(__uint_as_float(r[j + 1])), "f"(__uint_as_float(r[j + 2])), "f"(__uint_as_float(r[j + 3]))
                   : "memory");
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncol) asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + j), "f"(__uint_as_float(r[j])) : "memory");
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1)
xty_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                     const __grid_constant__ CUtensorMap tm_out, const XtyPairParams p) {
  using Cfg = XtyPairCfg;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* store_box = smem + kStages * Cfg::kStageBytes;      // 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_box + Cfg::kStoreBytes);
  uint64_t* full_bar = bars;                 // used in the leader only
  uint64_t* empty_bar = bars + kStages;      // both CTAs
  uint64_t* acc_full = bars + 2 * kStages;   // [2], both CTAs
  uint64_t* acc_empty = acc_full + 2;        // [2], used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const long long pair = blockIdx.x >> 1;
  const long long num_pairs = gridDim.x >> 1;
  const int blocks_mn = p.m_tiles * p.n_tiles;
  const long long units = static_cast<long long>(blocks_mn) * p.samples;
  const int kb_total = static_cast<int>((p.T + BK - 1) / BK);
  // unit -> (sample, tm, tn): sample-major, the index with fewer blocks innermost, dealt round-robin
  // to the pairs (neighbouring pairs then read adjacent column blocks of the same token rows)
  auto decode = [&](long long u, int& sample, int& tm, int& tn) {
    const bool n_inner = p.n_tiles <= p.m_tiles;
    const int n_in = n_inner ? p.n_tiles : p.m_tiles;
    sample = static_cast<int>(u / blocks_mn);
    const int r = static_cast<int>(u % blocks_mn);
    const int outer = r / n_in, in = r % n_in;
    tm = n_inner ? outer : in;
    tn = n_inner ? in : outer;
  };
  // row blocks (BK tokens) a unit contracts: the whole sample, or one split of the single sample
  auto k_range = [&](int sample, int& kb0, int& kb1) {
    if (!p.accumulate) { kb0 = 0; kb1 = kb_total; return; }
    kb0 = sample * p.kb_per_split;
    kb1 = kb0 + p.kb_per_split;
    if (kb1 > kb_total) kb1 = kb_total;
    if (kb0 > kb1) kb0 = kb1;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);    // 4 epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_y);
    if (p.tma_store) tma_prefetch_desc(&tm_out);
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
      for (long long u = pair; u < units && ok; u += num_pairs) {
        int sample, tm, tn;
        decode(u, sample, tm, tn);
        const int xblk = (tm * 2 * BM + static_cast<int>(rank) * BM) / 64;        // 64-column blocks
        const int yblk = (tn * BN + static_cast<int>(rank) * Cfg::BNH) / 64;
        const int z = p.accumulate ? 0 : p.sample0 + sample;
        int kb0, kb1;
        k_range(sample, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, 451)) { ok = false; break; }
          uint8_t* st = smem + stage * Cfg::kStageBytes;
          // the leader's barrier collects both CTAs' bytes
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          tma_load_4d_pair(st, &tm_x, bar, 0, kb * BK, xblk, z);
          tma_load_4d_pair(st + BM * BK * 2, &tm_y, bar, 0, kb * BK, yblk, z);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, 1, 1);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (long long u = pair; u < units && ok; u += num_pairs) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.err, 552)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t dst = tmem_base + acc * BN;
        int sample, tm, tn, kb0, kb1;
        decode(u, sample, tm, tn);
        k_range(sample, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.err, 553)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          // MN-major: LBO = distance between 64-column panels, SBO = 8 token rows
          const uint64_t adesc = make_smem_desc_sw128(sa, BK * 128, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sa + BM * BK * 2, BK * 128, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16_pair(dst, adesc + k * (16 * 128 / 16), bdesc + k * (16 * 128 / 16), idesc,
                           (kb == kb0 && k == 0) ? 0u : 1u);
          umma_commit_pair(&empty_bar[stage], 3);      // frees the stage in both CTAs
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&acc_full[acc], 3);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ column sums (warps 6-9, both CTAs)
    // Present only in launches that ask for them (320 threads).  Every unit adds its share of the
    // sample's token rows of the chosen operand's 256-column block to the sums: CTA r the 128
    // columns it also loads for the tensor core.
    float* red = reinterpret_cast<float*>(smem + kStages * Cfg::kStageBytes + Cfg::kStoreBytes + 1024 + 256);
    const int ct = static_cast<int>(threadIdx.x) - 192;
    for (long long u = pair; u < units; u += num_pairs) {
      int sample, tm, tn;
      decode(u, sample, tm, tn);
      // the units that share this (sample, column block) split the sample's token rows among them
      const int part = (p.cs_of == 1) ? tn : tm, parts = (p.cs_of == 1) ? p.n_tiles : p.m_tiles;
      const long long per = ((p.T + parts - 1) / parts + 7) / 8 * 8;
      const long long t0 = part * per;
      const long long t1 = (t0 + per < p.T) ? t0 + per : p.T;
      if (t0 >= t1) continue;
      const int cbase = ((p.cs_of == 1) ? tm : tn) * BN + static_cast<int>(rank) * 128;
      const long long s_idx = p.sample0 + sample;
      xty_colsum_128(p.cs_src + s_idx * p.T * p.cs_ld, t0, t1, p.cs_ld, cbase, p.cs_cols, red,
                     p.cs_out + s_idx * p.cs_cols, ct, 1);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-3, both CTAs)
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t boxes = 0;          // boxes handed to the copy engine so far (selects the staging buffer)
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    for (long long u = pair; u < units; u += num_pairs) {
      int sample, tm, tn;
      decode(u, sample, tm, tn);
      bool ok = mbar_wait_warp(&acc_full[acc], acc_phase, abort_flag, p.err, 154);
      // the staged store synchronises the four warps on a named barrier: they leave together
      if (p.tma_store) ok = named_bar_and(2, 128, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int tile128 = tm * 2 + static_cast<int>(rank);      // this CTA's 128-row tile
      if (p.accumulate) {
        int kb0, kb1;
        k_range(sample, kb0, kb1);
        const int m = tile128 * BM + static_cast<int>(threadIdx.x);
        const int n0 = tn * BN;
        const uint32_t t_acc = tmem_base + lane_base + acc * BN;
        const bool live = m < p.m_cols && kb0 < kb1;      // no row block: nothing was accumulated
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (n0 + c0 >= p.n_cols) break;
          uint32_t r[32];
          tmem_ld32(t_acc + c0, r);
          tmem_ld_wait();
          if (live)
            red_add_row32_pair(p.acc_ws + static_cast<long long>(m) * p.ld_acc + n0 + c0, r, p.n_cols - (n0 + c0));
        }
      } else if (tile128 < p.m_tiles128 && p.tma_store) {
        // Tile rows of 512 bytes lie 512 bytes apart: a warp-wide st.global touches 32 lines, and
        // its passes through the L1 data path compete with the column-sum warps' loads and the
        // operand traffic of the tensor core.  Instead every thread writes its row's 64 bytes into
        // a swizzled [128][32] box (conflict-free 16-byte stores) and the copy engine writes the
        // box out: 2.5 % off the call inside the GPT-2 step.  (Leaving the stores out altogether
        // makes the kernel 13 % faster: the 189 MB of tile writes themselves are what costs.)
        const uint32_t t_acc = tmem_base + lane_base + acc * BN;
        const int row = static_cast<int>(threadIdx.x);
        const int y0 = ((tile128 * p.n_tiles + tn) * p.samples + sample) * BM;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32, ++boxes) {
          uint32_t r[32];
          tmem_ld32(t_acc + c0, r);
          tmem_ld_wait();
          uint8_t* box = store_box + (boxes & 1) * Cfg::kStoreBoxBytes;
          // the store that read this buffer two boxes ago has finished reading it
          if (threadIdx.x == 0) bulk_wait_group_read<1>();
          named_bar_sync(2, 128);
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 hv =
                  __floats2bfloat162_rn(__uint_as_float(r[8 * ch + 2 * e]), __uint_as_float(r[8 * ch + 2 * e + 1]));
              w[e] = *reinterpret_cast<const uint32_t*>(&hv);
            }
            st_shared_v4(box + row * 64 + ((ch ^ ((row >> 1) & 3)) << 4), w[0], w[1], w[2], w[3]);
          }
          fence_proxy_async_smem();
          named_bar_sync(2, 128);
          if (threadIdx.x == 0) {
            tma_store_2d(&tm_out, box, c0, y0);
            bulk_commit_group();
          }
        }
      } else if (tile128 < p.m_tiles128) {
        const uint32_t t_acc = tmem_base + lane_base + acc * BN;
        const long long tbase =
            ((static_cast<long long>(tile128) * p.n_tiles + tn) * p.samples + sample) * (BM * BN) +
            static_cast<long long>(threadIdx.x) * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
          uint32_t r0[32], r1[32];
          tmem_ld32(t_acc + c0, r0);
          tmem_ld32(t_acc + c0 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t* r = h ? r1 : r0;
            if (p.v_is_f32) {
              float* dstp = static_cast<float*>(p.vgrad) + tbase + c0 + 32 * h;
#pragma unroll
              for (int q = 0; q < 4; ++q) st_global_v8_pair(dstp + 8 * q, &r[8 * q]);
            } else {
              uint32_t w[16];
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const __nv_bfloat162 hv = __floats2bfloat162_rn(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
                w[e] = *reinterpret_cast<const uint32_t*>(&hv);
              }
              __nv_bfloat16* dstp = static_cast<__nv_bfloat16*>(p.vgrad) + tbase + c0 + 32 * h;
              st_global_v8_pair(dstp, &w[0]);
              st_global_v8_pair(dstp + 16, &w[8]);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    // the boxes still in flight are written out before the CTA gives up its shared memory
    if (threadIdx.x == 0) bulk_wait_group<0>();
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

static int pair_kernel_smem_attr(const DeviceState* ds) {
  static bool attr_set[64] = {};
  if (!attr_set[ds->device]) {
    GB_CUDA_OK(cudaFuncSetAttribute(xty_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    XtyPairCfg::kSmemBytes));
    attr_set[ds->device] = true;
  }
  return GHOST_OK;
}

// Whether the device can hold at least one cluster of the pair kernel (asked once per device; a
// partitioned or otherwise restricted device may not): callers fall back to the single-CTA kernel.
bool xty_pair_usable(const DeviceState* ds) {
  static int state[64] = {};      // 0 unknown, 1 usable, -1 not
  if (ds->sm_count < 2) return false;
  int& st = state[ds->device];
  if (st == 0) {
    st = -1;
    if (pair_kernel_smem_attr(ds) == GHOST_OK) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2, 1, 1);
      cfg.blockDim = dim3(192, 1, 1);
      cfg.dynamicSmemBytes = XtyPairCfg::kSmemBytes;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, xty_gemm_pair_kernel, &cfg) == cudaSuccess && clusters > 0)
        st = 1;
      else
        (void)cudaGetLastError();
    }
  }
  return st == 1;
}

// X: [n_samples_total, T, m_cols], Y: [n_samples_total, T, n_cols] bf16, both column counts multiples
// of 64.  Writes the tiles of samples [sample0, sample0 + samples) to vgrad ([tile][samples][128][256]).
int launch_xty_pair_tiles(const void* X, const void* Y, long long n_samples_total, long long T, int m_cols,
                          int n_cols, long long ldx, long long ldy, int samples, int sample0, void* vgrad,
                          int v_is_f32, int colsum_of, float* colsum_out, const DeviceState* ds, cudaStream_t st) {
  using Cfg = XtyPairCfg;
  XtyPairParams p;
  p.m_cols = m_cols;
  p.n_cols = n_cols;
  p.m_tiles128 = ceil_div(m_cols, 128);
  p.m_tiles = ceil_div(m_cols, 256);
  p.n_tiles = ceil_div(n_cols, 256);
  p.samples = samples;
  p.sample0 = sample0;
  p.T = T;
  p.vgrad = vgrad;
  p.v_is_f32 = v_is_f32;
  // bf16 tiles go out through the copy engine (row counts up to 2^31 keep the box coordinate an int)
  const unsigned long long out_rows = static_cast<unsigned long long>(p.m_tiles128) * p.n_tiles * samples * Cfg::BM;
  p.tma_store = (!v_is_f32 && out_rows < (1ull << 31)) ? 1 : 0;
  p.accumulate = 0;
  p.kb_per_split = 0;
  p.acc_ws = nullptr;
  p.ld_acc = 0;
  p.cs_of = (colsum_out != nullptr) ? colsum_of : 0;
  p.cs_src = static_cast<const __nv_bfloat16*>(p.cs_of == 1 ? X : Y);
  p.cs_ld = (p.cs_of == 1) ? ldx : ldy;
  p.cs_cols = (p.cs_of == 1) ? m_cols : n_cols;
  p.cs_out = colsum_out;
  p.err = ds->err_word;
  if (p.cs_of)
    GB_CUDA_OK(cudaMemsetAsync(colsum_out + static_cast<long long>(sample0) * p.cs_cols, 0,
                               sizeof(float) * static_cast<size_t>(samples) * p.cs_cols, st));
  CUtensorMap tx, ty;
  int rc;
  if ((rc = make_tmap_bf16_blocks(&tx, X, n_samples_total, T, m_cols, ldx, Cfg::BK, Cfg::BM / 64)) != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_blocks(&ty, Y, n_samples_total, T, n_cols, ldy, Cfg::BK, Cfg::BNH / 64)) != GHOST_OK) return rc;
  CUtensorMap tout = tx;
  if (p.tma_store && (rc = make_tmap_bf16_store_2d(&tout, vgrad, out_rows, Cfg::BN, Cfg::BM)) != GHOST_OK) return rc;
  if ((rc = pair_kernel_smem_attr(ds)) != GHOST_OK) return rc;
  const long long units = static_cast<long long>(p.m_tiles) * p.n_tiles * samples;
  long long pairs = ds->sm_count / 2;
  if (pairs > units) pairs = units;
  xty_gemm_pair_kernel<<<static_cast<int>(2 * pairs), p.cs_of ? 320 : 192, Cfg::kSmemBytes, st>>>(tx, ty, tout, p);
  count_launch();
  return post_launch("xty_gemm_pair_kernel");
}

// Train-gradient pass: acc_ws[m_cols, ld_acc] (fp32, zeroed by the caller) += X^T Y over n_rows token
// rows.  Both column counts are multiples of 64.
int launch_xty_pair_wgrad(const void* X, const void* Y, long long n_rows, int m_cols, int n_cols, long long ldx,
                          long long ldy, float* acc_ws, long long ld_acc, const DeviceState* ds,
                          cudaStream_t st) {
  using Cfg = XtyPairCfg;
  XtyPairParams p;
  p.m_cols = m_cols;
  p.n_cols = n_cols;
  p.m_tiles128 = ceil_div(m_cols, 128);
  p.m_tiles = ceil_div(m_cols, 256);
  p.n_tiles = ceil_div(n_cols, 256);
  p.sample0 = 0;
  p.T = n_rows;
  p.vgrad = nullptr;
  p.v_is_f32 = 0;
  p.tma_store = 0;
  p.accumulate = 1;
  p.acc_ws = acc_ws;
  p.ld_acc = ld_acc;
  p.cs_of = 0;
  p.cs_src = nullptr;
  p.cs_ld = 0;
  p.cs_cols = 0;
  p.cs_out = nullptr;
  p.err = ds->err_word;
  const long long pairs_max = ds->sm_count / 2;
  const int kb = static_cast<int>(ceil_div(n_rows, static_cast<long long>(Cfg::BK)));
  const long long blocks = static_cast<long long>(p.m_tiles) * p.n_tiles;
  // Split-K factor with the shortest critical path: ceil(units / pairs) rounds of (row blocks per
  // split + a fixed cost per unit for the accumulator hand-over and the red.add epilogue).
  int splits = 1;
  long long best = -1;
  for (int s = 1; s <= 64 && s <= kb; ++s) {
    const long long rounds = (blocks * s + pairs_max - 1) / pairs_max;
    const long long cost = rounds * (ceil_div(kb, s) + 32);
    if (best < 0 || cost < best) { best = cost; splits = s; }
  }
  p.kb_per_split = ceil_div(kb, splits);
  p.samples = ceil_div(kb, p.kb_per_split);
  CUtensorMap tx, ty;
  int rc;
  if ((rc = make_tmap_bf16_blocks(&tx, X, 1, n_rows, m_cols, ldx, Cfg::BK, Cfg::BM / 64)) != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_blocks(&ty, Y, 1, n_rows, n_cols, ldy, Cfg::BK, Cfg::BNH / 64)) != GHOST_OK) return rc;
  if ((rc = pair_kernel_smem_attr(ds)) != GHOST_OK) return rc;
  const long long units = blocks * p.samples;
  const long long pairs = pairs_max < units ? pairs_max : units;
  xty_gemm_pair_kernel<<<static_cast<int>(2 * pairs), 192, Cfg::kSmemBytes, st>>>(tx, ty, tx, p);
  count_launch();
  return post_launch("xty_gemm_pair_kernel");
}

}  // namespace gb
