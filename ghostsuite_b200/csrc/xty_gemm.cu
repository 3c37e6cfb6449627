// xty_gemm: token-contracted outer-product GEMMs  D[m, n] = sum_rows X[row, m] * Y[row, n].
//
// X and Y are token-major bf16 matrices ([samples, T, cols]); the contraction runs over token rows,
// so both operands are "MN-major" for tcgen05: a shared-memory stage holds 64 token rows, and each
// 64-column slab of them is one TMA box (64 rows x 128 bytes, 128B swizzle).  Three uses share the
// mainloop and differ in the epilogue:
//
//   kEpiAccumulate  train-gradient recovery (ghostEngines/supported_layers_grad_samplers_dotprod.py
//                   :168 and :502): contraction over all train tokens, optionally split across
//                   CTAs; partial tiles are added into an fp32 workspace with red.global.add.
//   kEpiStore       per-validation-sample weight gradients V[v] written to a workspace
//                   (per-sample form of :133-134).
//   kEpiStoreTiles  per-sample weight-gradient tiles (train and validation samples alike) written
//                   tile-major as bf16 (fp32 for split fp32 inputs); tile_dot.cu then contracts
//                   them into the [n_val, n_train] matrix and the train-gradient sum in one
//                   streaming pass (per-sample form of :133-135).
//
// Linear weights are [d_out, d_in]: X = G (out-grad), Y = A (activations).  HF Conv1D weights are
// [d_in, d_out]: X = A, Y = G.  No transposes are materialised.
//
// CTA layout (192 threads, persistent): warps 0-3 epilogue, warp 4 TMA producer, warp 5 TMEM
// allocator + MMA issuer.  128 x 256 fp32 accumulator, double-buffered in TMEM (512 columns).
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "xty_colsum.cuh"

namespace gb {

enum { kEpiAccumulate = 0, kEpiStore = 1, kEpiStoreTiles = 2 };

struct XtyParams {
  int mode;
  int m_cols, n_cols;        // output extent (X columns, Y columns)
  int m_tiles, n_tiles;
  int samples;               // samples contracted separately (1 for plain train-gradient recovery)
  int sample0;               // first sample (z coordinate offset into the tensor maps)
  long long T;               // token rows per sample
  int k_splits;              // kEpiAccumulate: CTAs sharing one output tile
  int kb_per_split;          // 64-row blocks per split
  int units_per_cta;         // each CTA takes a contiguous range of units
  // kEpiAccumulate: fp32 [m_cols, ld_acc] accumulation workspace
  float* acc_ws;
  long long ld_acc;
  // kEpiStore: row-major [sample][m_cols][ld_v]; kEpiStoreTiles: tile-major [tile][sample][128][256]
  void* vgrad;
  long long ld_v;
  int v_is_f32;
  int sample_major;          // unit order (sample, tile), dealt round-robin to the CTAs; needs k_splits == 1
  // per-sample column sums of one operand (bias terms), taken by four extra warps that read the
  // operand rows through L2: 0 = none, 1 = X, 2 = Y; out [all samples, cols of that operand] fp32
  int colsum_of;
  float* colsum_out;
  const __nv_bfloat16* cs_src;   // that operand, [all samples, T, cols], row pitch cs_ld
  long long cs_ld;
  int blocked_x, blocked_y;  // operand map is the blocked 4-D form: one TMA per stage instead of one per 64 columns
  int* err;
};

struct XtyCfg {
  static constexpr int BM = 128, BN = 256, BK = 64;
  static constexpr int kStageBytes = (BM + BN) * BK * 2;   // 48 KB
  static constexpr int kStages = 4;
  static constexpr int kColsumBytes = 8 * 128 * 4;          // reduction scratch of the column-sum warps
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + kColsumBytes;
};

// one 256-bit store (the address must be 32-byte aligned)
__device__ __forceinline__ void st_global_v8(void* addr, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(addr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void red_add_f32(float* addr, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
// 32 consecutive accumulator columns of one output row -> fp32 workspace (16-byte aligned rows)
__device__ __forceinline__ void red_add_row32(float* dst, const uint32_t (&r)[32], int ncol) {
  if (ncol >= 32) {
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      red_add_f32x4(dst + j, __uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                    __uint_as_float(r[j + 3]));
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncol) red_add_f32(dst + j, __uint_as_float(r[j]));
  }
}

template <bool kColsum>
__global__ void __launch_bounds__(kColsum ? 320 : 192, 1)
xty_gemm_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                const XtyParams p) {
  using Cfg = XtyCfg;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* acc_full = bars + 2 * kStages;     // [2]
  uint64_t* acc_empty = acc_full + 2;          // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_mn = p.m_tiles * p.n_tiles;
  // unit -> (tile, sample, split).  Plain order: tile-major, samples and splits inside.  Tile-store
  // mode walks (sample, outer tile index, inner tile index) instead, the inner index being the one
  // with fewer tiles: neighbouring units share the tile of the wider operand.
  const long long units = static_cast<long long>(tiles_mn) * p.samples * p.k_splits;
  const int kb_sample = static_cast<int>((p.T + BK - 1) / BK);
  // plain order: a contiguous range per CTA; sample-major order: units dealt round-robin, so that
  // at any time the CTAs work on neighbouring tiles of the same sample (their operand rows are
  // adjacent in HBM and shared through L2)
  const long long u_step = p.sample_major ? gridDim.x : 1;
  const long long u_begin = p.sample_major ? blockIdx.x : static_cast<long long>(blockIdx.x) * p.units_per_cta;
  const long long u_end = p.sample_major ? units
                          : ((u_begin + p.units_per_cta < units) ? u_begin + p.units_per_cta : units);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_y);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  auto decode = [&](long long u, int& tile, int& sample, int& kb0, int& kb1) {
    if (p.sample_major) {
      const bool n_inner = p.n_tiles <= p.m_tiles;
      const int n_in = n_inner ? p.n_tiles : p.m_tiles;
      sample = static_cast<int>(u / tiles_mn);
      const int r = static_cast<int>(u % tiles_mn);
      const int outer = r / n_in, in = r % n_in;
      tile = n_inner ? outer * p.n_tiles + in : in * p.n_tiles + outer;
      kb0 = 0;
      kb1 = kb_sample;
      return;
    }
    const int inner = p.samples * p.k_splits;
    tile = static_cast<int>(u / inner);
    const int r = static_cast<int>(u % inner);
    sample = r / p.k_splits;
    const int split = r % p.k_splits;
    kb0 = split * p.kb_per_split;
    kb1 = kb0 + p.kb_per_split;
    if (kb1 > kb_sample) kb1 = kb_sample;
    if (kb0 > kb1) kb0 = kb1;
  };

  if (warp == 4) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long u = u_begin; u < u_end && ok; u += u_step) {
        int tile, sample, kb0, kb1;
        decode(u, tile, sample, kb0, kb1);
        const int m0 = (tile / p.n_tiles) * BM;
        const int n0 = (tile % p.n_tiles) * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, 411)) { ok = false; break; }
          uint8_t* st = smem + stage * Cfg::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          const int row = kb * BK;
          const int z = p.sample0 + sample;
          // Every TMA instruction costs the issuing thread on the order of 100 cycles whatever its
          // size, and six of them per stage would take longer than the stage's MMAs.
          if (p.blocked_x) {
            tma_load_4d(st, &tm_x, &full_bar[stage], 0, row, m0 / 64, z);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(st + j * (BK * 128), &tm_x, &full_bar[stage], m0 + j * 64, row, z);
          }
          if (p.blocked_y) {
            tma_load_4d(st + BM * BK * 2, &tm_y, &full_bar[stage], 0, row, n0 / 64, z);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(st + BM * BK * 2 + j * (BK * 128), &tm_y, &full_bar[stage], n0 + j * 64, row, z);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (long long u = u_begin; u < u_end && ok; u += u_step) {
        int tile, sample, kb0, kb1;
        decode(u, tile, sample, kb0, kb1);
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.err, 512)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t dst = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.err, 513)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          // MN-major: LBO = distance between 64-column slabs (one TMA box), SBO = 8 token rows
          const uint64_t adesc = make_smem_desc_sw128(sa, BK * 128, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sa + BM * BK * 2, BK * 128, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16(dst, adesc + k * (16 * 128 / 16), bdesc + k * (16 * 128 / 16), idesc,
                      (kb == kb0 && k == 0) ? 0u : 1u);
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (kColsum && warp >= 6) {
    // ---------------------------------------------------------------- column sums (warps 6-9)
    // Every unit adds its share of the sample's token rows to the sums of its column block; see
    // xty_colsum.cuh.
    float* red = reinterpret_cast<float*>(smem + kStages * Cfg::kStageBytes + 1024 + 256);
    const int ct = static_cast<int>(threadIdx.x) - 192;
    const bool of_y = p.colsum_of == 2;
    const int total_cols = of_y ? p.n_cols : p.m_cols;
    for (long long u = u_begin; u < u_end; u += u_step) {
      int tile, sample, kb0, kb1;
      decode(u, tile, sample, kb0, kb1);
      const int tm = tile / p.n_tiles, tn = tile % p.n_tiles;
      // the units that share this (sample, column block) split the sample's token rows among them
      const int part = of_y ? tm : tn, parts = of_y ? p.m_tiles : p.n_tiles;
      const long long per = ((p.T + parts - 1) / parts + 7) / 8 * 8;
      const long long t0 = part * per;
      const long long t1 = (t0 + per < p.T) ? t0 + per : p.T;
      if (t0 >= t1) continue;
      const long long s_idx = p.sample0 + sample;
      const int width = of_y ? BN : BM;
      for (int half = 0; half < width; half += 128)
        xty_colsum_128(p.cs_src + s_idx * p.T * p.cs_ld, t0, t1, p.cs_ld, (of_y ? tn * BN : tm * BM) + half, total_cols,
                       red, p.colsum_out + s_idx * total_cols, ct, 1);
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    for (long long u = u_begin; u < u_end; u += u_step) {
      int tile, sample, kb0, kb1;
      decode(u, tile, sample, kb0, kb1);
      const int m0 = (tile / p.n_tiles) * BM;
      const int n0 = (tile % p.n_tiles) * BN;
      if (!mbar_wait_warp(&acc_full[acc], acc_phase, abort_flag, p.err, 114)) break;
      tc_fence_after_sync();
      const int m = m0 + threadIdx.x;
      const bool m_ok = m < p.m_cols;
      const uint32_t t_acc = tmem_base + lane_base + acc * BN;
      const bool empty_k = (kb0 >= kb1);   // nothing was accumulated: the tile is all zero

      if (p.mode == kEpiAccumulate) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (n0 + c0 >= p.n_cols) break;
          uint32_t r[32];
          tmem_ld32(t_acc + c0, r);
          tmem_ld_wait();
          if (m_ok && !empty_k)
            red_add_row32(p.acc_ws + static_cast<long long>(m) * p.ld_acc + n0 + c0, r, p.n_cols - (n0 + c0));
        }
      } else if (p.mode == kEpiStore) {
        const long long vbase = (static_cast<long long>(sample) * p.m_cols + m) * p.ld_v;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (n0 + c0 >= p.ld_v) break;
          uint32_t r[32];
          tmem_ld32(t_acc + c0, r);
          tmem_ld_wait();
          if (m_ok) {
            // columns in [n_cols, ld_v) are written too (their accumulators are exact zeros from
            // the TMA zero fill) so that the vector loads of the dot epilogue never see garbage
            if (p.v_is_f32) {
              float* dst = static_cast<float*>(p.vgrad) + vbase + n0 + c0;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + c0 + j < p.ld_v) dst[j] = empty_k ? 0.f : __uint_as_float(r[j]);
            } else {
              __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.vgrad) + vbase + n0 + c0;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + c0 + j < p.ld_v)
                  dst[j] = __float2bfloat16_rn(empty_k ? 0.f : __uint_as_float(r[j]));
            }
          }
        }
      } else {
        // kEpiStoreTiles: the whole 128 x 256 tile (zero padded), tile-major:
        //   dst[(tile * samples + sample)][row][col], one 512- or 1024-byte row per thread
        const long long tbase = (static_cast<long long>(tile) * p.samples + sample) * (BM * BN) +
                                static_cast<long long>(threadIdx.x) * BN;
        // two TMEM loads in flight per wait, 32-byte stores (every store fills whole sectors)
        auto store32 = [&](int c0, uint32_t (&r)[32]) {
          if (empty_k) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
          if (p.v_is_f32) {
            float* dst = static_cast<float*>(p.vgrad) + tbase + c0;
#pragma unroll
            for (int q = 0; q < 4; ++q) st_global_v8(dst + 8 * q, &r[8 * q]);
          } else {
            uint32_t w[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
              w[e] = *reinterpret_cast<const uint32_t*>(&h);
            }
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.vgrad) + tbase + c0;
            st_global_v8(dst, &w[0]);
            st_global_v8(dst + 16, &w[8]);
          }
        };
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
          uint32_t r0[32], r1[32];
          tmem_ld32(t_acc + c0, r0);
          tmem_ld32(t_acc + c0 + 32, r1);
          tmem_ld_wait();
          store32(c0, r0);
          store32(c0 + 32, r1);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// finalize: out = (accumulate ? out : 0) + scale * ws, cast to the parameter dtype
template <typename OutT>
__global__ void xty_finalize_kernel(const float* __restrict__ ws, long long ld_ws, OutT* __restrict__ out,
                                    int rows, int cols, float scale, int accumulate) {
  const long long n = static_cast<long long>(rows) * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / cols), c = static_cast<int>(i % cols);
    float v = ws[static_cast<long long>(r) * ld_ws + c] * scale;
    if (accumulate) v += static_cast<float>(out[i]);
    out[i] = static_cast<OutT>(v);
  }
}

// CTA-pair variant of the tile-store pass (xty_gemm_pair.cu)
int launch_xty_pair_tiles(const void* X, const void* Y, long long n_samples_total, long long T, int m_cols,
                          int n_cols, long long ldx, long long ldy, int samples, int sample0, void* vgrad,
                          int v_is_f32, int colsum_of, float* colsum_out, const DeviceState* ds, cudaStream_t st);
int launch_xty_pair_wgrad(const void* X, const void* Y, long long n_rows, int m_cols, int n_cols, long long ldx,
                          long long ldy, float* acc_ws, long long ld_acc, const DeviceState* ds, cudaStream_t st);
bool xty_pair_usable(const DeviceState* ds);
static int g_wgrad_pair_mode = 1;      // same meaning as below
static int g_persample_pair_mode = 1;  // 0 off, 1 where no half of a pair would idle, 2 wherever applicable

// Operand maps: the blocked form (one TMA instruction per operand and stage) when the column count
// is a multiple of 64, else one box per 64 columns with the tail zero-filled by the bounds check.
static int make_xty_maps(CUtensorMap* tx, CUtensorMap* ty, XtyParams& p, const void* X, const void* Y,
                         long long samples, long long rows, long long ldx, long long ldy) {
  int rc;
  p.blocked_x = (p.m_cols % 64 == 0) ? 1 : 0;
  p.blocked_y = (p.n_cols % 64 == 0) ? 1 : 0;
  rc = p.blocked_x ? make_tmap_bf16_blocks(tx, X, samples, rows, p.m_cols, ldx, XtyCfg::BK, XtyCfg::BM / 64)
                   : make_tmap_bf16_3d(tx, X, samples, rows, p.m_cols, ldx, XtyCfg::BK);
  if (rc != GHOST_OK) return rc;
  return p.blocked_y ? make_tmap_bf16_blocks(ty, Y, samples, rows, p.n_cols, ldy, XtyCfg::BK, XtyCfg::BN / 64)
                     : make_tmap_bf16_3d(ty, Y, samples, rows, p.n_cols, ldy, XtyCfg::BK);
}

static int launch_xty(const CUtensorMap& tx, const CUtensorMap& ty, XtyParams p,
                      const DeviceState* ds, cudaStream_t st) {
  static bool attr_set[64] = {};
  if (!attr_set[ds->device]) {
    GB_CUDA_OK(cudaFuncSetAttribute(xty_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    XtyCfg::kSmemBytes));
    GB_CUDA_OK(cudaFuncSetAttribute(xty_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    XtyCfg::kSmemBytes));
    attr_set[ds->device] = true;
  }
  const long long units = static_cast<long long>(p.m_tiles) * p.n_tiles * p.samples * p.k_splits;
  int grid = static_cast<int>(units < ds->sm_count ? units : ds->sm_count);
  p.units_per_cta = static_cast<int>((units + grid - 1) / grid);
  if (!p.sample_major) grid = static_cast<int>((units + p.units_per_cta - 1) / p.units_per_cta);
  if (p.colsum_of != 0 && p.colsum_out != nullptr) {
    // the column-sum warps add into the output: zero the rows of this launch's samples first
    const int cs_cols = p.colsum_of == 2 ? p.n_cols : p.m_cols;
    GB_CUDA_OK(cudaMemsetAsync(p.colsum_out + static_cast<long long>(p.sample0) * cs_cols, 0,
                               sizeof(float) * static_cast<size_t>(p.samples) * cs_cols, st));
    xty_gemm_kernel<true><<<grid, 320, XtyCfg::kSmemBytes, st>>>(tx, ty, p);
  }
  else
    xty_gemm_kernel<false><<<grid, 192, XtyCfg::kSmemBytes, st>>>(tx, ty, p);
  count_launch();
  return post_launch("xty_gemm_kernel");
}

int finalize_xty(const float* ws, long long ld_ws, void* out, int out_is_f32, int rows, int cols,
                 float scale, int accumulate, cudaStream_t st) {
  const long long n = static_cast<long long>(rows) * cols;
  const int grid = static_cast<int>(n / 256 + 1 < 148 * 8 ? n / 256 + 1 : 148 * 8);
  if (out_is_f32)
    xty_finalize_kernel<float><<<grid, 256, 0, st>>>(ws, ld_ws, static_cast<float*>(out), rows, cols, scale, accumulate);
  else
    xty_finalize_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(ws, ld_ws, static_cast<__nv_bfloat16*>(out), rows, cols, scale, accumulate);
  count_launch();
  return post_launch("xty_finalize_kernel");
}

}  // namespace gb

using namespace gb;

static inline long long round_up(long long x, long long m) { return (x + m - 1) / m * m; }

// a pair covers two 128-row tiles of X's columns: with an odd tile count the last pair's second CTA
// idles, which costs more than the pair saves unless there are many tiles
static bool pair_kernel_fits(int mode, int m_cols, int n_cols) {
  if (mode == 0 || m_cols % 64 != 0 || n_cols % 64 != 0) return false;
  const int m_tiles128 = (m_cols + 127) / 128;
  return mode == 2 || m_tiles128 % 2 == 0 || m_tiles128 >= 15;
}

extern "C" int ghost_set_wgrad_pair_mode(int mode) {
  if (mode < 0 || mode > 2) return GHOST_ERR_INVALID;
  g_wgrad_pair_mode = mode;
  return GHOST_OK;
}

extern "C" long long ghost_wgrad_workspace_bytes(int m_cols, int n_cols) {
  return static_cast<long long>(m_cols) * round_up(n_cols, 4) * 4;
}

// D[m_cols, n_cols] = scale * sum_{rows < n_rows} X[row, :]^T Y[row, :]
extern "C" int ghost_wgrad_bf16(const void* X, const void* Y, long long n_rows, int m_cols, int n_cols,
                                long long ldx, long long ldy, float scale, int accumulate, void* out,
                                int out_is_f32, void* ws, long long ws_bytes, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(X && Y && out && ws, "ghost_wgrad_bf16: null pointer");
  GB_REQUIRE(n_rows > 0 && m_cols > 0 && n_cols > 0, "ghost_wgrad_bf16: empty dimension");
  GB_REQUIRE(n_rows < (1ll << 31) - 64, "ghost_wgrad_bf16: more than 2^31 token rows");
  GB_REQUIRE(ws_bytes >= ghost_wgrad_workspace_bytes(m_cols, n_cols), "ghost_wgrad_bf16: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  XtyParams p = {};
  p.mode = kEpiAccumulate;
  p.m_cols = m_cols;
  p.n_cols = n_cols;
  p.m_tiles = ceil_div(m_cols, XtyCfg::BM);
  p.n_tiles = ceil_div(n_cols, XtyCfg::BN);
  p.samples = 1;
  p.sample0 = 0;
  p.T = n_rows;
  const int kb = ceil_div(n_rows, XtyCfg::BK);
  const int tiles = p.m_tiles * p.n_tiles;
  // Split-K factor: the CTAs run ceil(units / SMs) rounds of (k-blocks per split + a fixed cost per
  // unit for the accumulator hand-over and the red.add epilogue, measured at about 64 k-blocks' worth); take
  // the factor with the shortest critical path.
  int splits = 1;
  long long best = -1;
  for (int s = 1; s <= 64 && s <= kb; ++s) {
    const long long units = static_cast<long long>(tiles) * s;
    const long long rounds = (units + ds->sm_count - 1) / ds->sm_count;
    const long long cost = rounds * (ceil_div(kb, s) + 64);
    if (best < 0 || cost < best) { best = cost; splits = s; }
  }
  p.kb_per_split = ceil_div(kb, splits);
  p.k_splits = ceil_div(kb, p.kb_per_split);
  p.acc_ws = static_cast<float*>(ws);
  p.ld_acc = round_up(n_cols, 4);
  p.err = ds->err_word;
  CUtensorMap tx, ty;
  int rc;
  if ((rc = make_xty_maps(&tx, &ty, p, X, Y, 1, n_rows, ldx, ldy)) != GHOST_OK) return rc;
  GB_CUDA_OK(cudaMemsetAsync(ws, 0, static_cast<size_t>(m_cols) * p.ld_acc * 4, st));
  if (pair_kernel_fits(g_wgrad_pair_mode, m_cols, n_cols) && p.blocked_x && p.blocked_y && xty_pair_usable(ds))
    rc = launch_xty_pair_wgrad(X, Y, n_rows, m_cols, n_cols, ldx, ldy, p.acc_ws, p.ld_acc, ds, st);
  else
    rc = launch_xty(tx, ty, p, ds, st);
  if (rc != GHOST_OK) return rc;
  return finalize_xty(p.acc_ws, p.ld_acc, out, out_is_f32, m_cols, n_cols, scale, accumulate, st);
}

namespace gb {
int launch_tile_dot(const void* V, int v_samples, int v_off, const void* W, int w_samples, int is_f32,
                    long long tiles, int n_val, int n_grp, int b0, int n_train, float scale, float* M,
                    float* sum, int sum_init, void* out, int out_is_f32, int out_accumulate, int m_cols,
                    int n_cols, int n_tiles_n, float out_scale, const DeviceState* ds, cudaStream_t st,
                    int v_per_rank = 0);
int launch_tile_sum_finalize(const float* sum, int n_tiles_n, void* out, int out_is_f32, int rows, int cols,
                             float scale, int accumulate, const DeviceState* ds, cudaStream_t st);
}

// Workspace of the per-sample path: fp32 tile-major train-gradient sum, validation tiles, and the
// tiles of one group of train samples.  The group size is the largest that keeps the workspace
// under `budget_bytes` (at least one sample).
static const long long kTileElems = 128 * 256;
static int persample_group(int n_train, int n_val, long long tiles, int esize, long long budget_bytes) {
  const long long per_sample = tiles * kTileElems * esize;
  long long g = (budget_bytes - tiles * kTileElems * 4) / per_sample - n_val;
  if (g < 1) g = 1;
  if (g > n_train) g = n_train;
  return static_cast<int>(g);
}
static long long kPersampleBudget = 12ll << 30;

extern "C" int ghost_set_persample_budget_bytes(long long bytes) {
  GB_REQUIRE(bytes >= (1ll << 20), "ghost_set_persample_budget_bytes: at least 1 MiB");
  kPersampleBudget = bytes;
  return GHOST_OK;
}

extern "C" long long ghost_persample_workspace_bytes(int n_train, int n_val, int m_cols, int n_cols, int v_is_f32) {
  const long long tiles = static_cast<long long>(ceil_div(m_cols, XtyCfg::BM)) * ceil_div(n_cols, XtyCfg::BN);
  const int esize = v_is_f32 ? 4 : 2;
  const int g = persample_group(n_train, n_val, tiles, esize, kPersampleBudget);
  return tiles * kTileElems * 4 + (static_cast<long long>(n_val) + g) * tiles * kTileElems * esize + 512;
}

extern "C" int ghost_set_persample_pair_mode(int mode) {
  if (mode < 0 || mode > 2) return GHOST_ERR_INVALID;
  g_persample_pair_mode = mode;
  return GHOST_OK;
}

// Per-sample-gradient path.  X, Y: [n_train + n_val, T, cols] (train first).  Produces
// M[v, b] = dot_scale * <X_v^T Y_v, X_b^T Y_b> and, if grad_out != null, the train gradient
// grad_scale * sum_b X_b^T Y_b (written or accumulated, cast to the parameter dtype).
extern "C" int ghost_persample_dot_bf16(const void* X, const void* Y, int n_train, int n_val, long long T,
                                        int m_cols, int n_cols, long long ldx, long long ldy,
                                        float dot_scale, float* M_out, int v_is_f32, void* grad_out,
                                        int grad_is_f32, float grad_scale, int grad_accumulate,
                                        int colsum_of, float* colsum_out,
                                        void* ws, long long ws_bytes, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(X && Y && M_out && ws, "ghost_persample_dot_bf16: null pointer");
  GB_REQUIRE(colsum_of >= 0 && colsum_of <= 2 && (colsum_of == 0 || colsum_out != nullptr),
             "ghost_persample_dot_bf16: colsum_of must be 0, 1 (X) or 2 (Y) with an output buffer");
  GB_REQUIRE(n_train > 0, "No training samples to compute dot product, check batch sizes.");
  GB_REQUIRE(n_val > 0 && T > 0 && m_cols > 0 && n_cols > 0, "ghost_persample_dot_bf16: empty dimension");
  GB_REQUIRE(T < (1ll << 31) - 64, "ghost_persample_dot_bf16: T too large");
  GB_REQUIRE(ws_bytes >= ghost_persample_workspace_bytes(n_train, n_val, m_cols, n_cols, v_is_f32),
             "ghost_persample_dot_bf16: workspace too small");
  GB_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 255u) == 0, "ghost_persample_dot_bf16: workspace must be 256-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int esize = v_is_f32 ? 4 : 2;
  XtyParams p = {};
  p.mode = kEpiStoreTiles;
  p.m_cols = m_cols;
  p.n_cols = n_cols;
  p.m_tiles = ceil_div(m_cols, XtyCfg::BM);
  p.n_tiles = ceil_div(n_cols, XtyCfg::BN);
  p.T = T;
  p.k_splits = 1;
  p.sample_major = 1;
  p.kb_per_split = ceil_div(T, XtyCfg::BK);
  p.v_is_f32 = v_is_f32;
  p.colsum_of = colsum_of;
  p.colsum_out = colsum_out;
  p.cs_src = static_cast<const __nv_bfloat16*>(colsum_of == 1 ? X : Y);
  p.cs_ld = (colsum_of == 1) ? ldx : ldy;
  p.err = ds->err_word;
  const long long tiles = static_cast<long long>(p.m_tiles) * p.n_tiles;
  const int group = persample_group(n_train, n_val, tiles, esize, kPersampleBudget);
  float* sum = static_cast<float*>(ws);
  uint8_t* vws = static_cast<uint8_t*>(ws) + tiles * kTileElems * 4;
  uint8_t* wws = vws + static_cast<long long>(n_val) * tiles * kTileElems * esize;
  CUtensorMap tx, ty;
  int rc;
  const long long N = static_cast<long long>(n_train) + n_val;
  if ((rc = make_xty_maps(&tx, &ty, p, X, Y, N, T, ldx, ldy)) != GHOST_OK) return rc;
  GB_CUDA_OK(cudaMemsetAsync(M_out, 0, sizeof(float) * static_cast<size_t>(n_val) * n_train, st));
  // tile pass: the CTA-pair kernel when it is selected and applicable, else the single-CTA kernel
  const bool use_pair = pair_kernel_fits(g_persample_pair_mode, m_cols, n_cols) && p.blocked_x && p.blocked_y &&
                        xty_pair_usable(ds);
  auto tile_pass = [&](const XtyParams& q) -> int {
    if (use_pair)
      return launch_xty_pair_tiles(X, Y, N, T, m_cols, n_cols, ldx, ldy, q.samples, q.sample0, q.vgrad,
                                   v_is_f32, colsum_of, colsum_out, ds, st);
    return launch_xty(tx, ty, q, ds, st);
  };
  if (group == n_train) {
    // everything fits: one GEMM pass over all samples (train first, validation last) into one
    // [tile][N][32768] buffer, one streaming pass over it
    p.samples = static_cast<int>(N);
    p.sample0 = 0;
    p.vgrad = vws;
    if ((rc = tile_pass(p)) != GHOST_OK) return rc;
    // With a single group the streaming kernel can write the train gradient itself (scaled, in the
    // parameter dtype): no fp32 sum buffer, no finalize pass.  A bf16 output is only written
    // directly when one 32-sample block covers the batch, so it is rounded once.
    const bool direct = grad_out && (grad_is_f32 || n_train <= 32);
    if ((rc = launch_tile_dot(vws, static_cast<int>(N), n_train, vws, static_cast<int>(N), v_is_f32, tiles,
                              n_val, n_train, 0, n_train, dot_scale, M_out,
                              (grad_out && !direct) ? sum : nullptr, 1, direct ? grad_out : nullptr,
                              grad_is_f32, grad_accumulate, m_cols, n_cols, p.n_tiles, grad_scale, ds,
                              st)) != GHOST_OK)
      return rc;
    if (direct || !grad_out) return GHOST_OK;
  } else {
    // validation tiles once, then the train samples one group at a time
    p.samples = n_val;
    p.sample0 = n_train;
    p.vgrad = vws;
    if ((rc = tile_pass(p)) != GHOST_OK) return rc;
    for (int b0 = 0; b0 < n_train; b0 += group) {
      const int g = (n_train - b0 < group) ? n_train - b0 : group;
      p.samples = g;
      p.sample0 = b0;
      p.vgrad = wws;
      if ((rc = tile_pass(p)) != GHOST_OK) return rc;
      if ((rc = launch_tile_dot(vws, n_val, 0, wws, g, v_is_f32, tiles, n_val, g, b0, n_train, dot_scale,
                                M_out, grad_out ? sum : nullptr, b0 == 0 ? 1 : 0, nullptr, 0, 0, m_cols,
                                n_cols, p.n_tiles, 1.f, ds, st)) != GHOST_OK)
        return rc;
    }
  }
  if (grad_out)
    return launch_tile_sum_finalize(sum, p.n_tiles, grad_out, grad_is_f32, m_cols, n_cols, grad_scale,
                                    grad_accumulate, ds, st);
  return GHOST_OK;
}

// ---- the two passes as separate calls ---------------------------------------------------------------
// For callers that put something between the passes: a data-parallel run whose ranks each hold a
// part of the validation batch computes its own validation tiles, all-gathers them, and only then
// contracts them with its train tiles.

extern "C" long long ghost_persample_tiles_bytes(int samples, int m_cols, int n_cols) {
  if (samples <= 0 || m_cols <= 0 || n_cols <= 0) return 0;
  const long long tiles = static_cast<long long>(ceil_div(m_cols, XtyCfg::BM)) * ceil_div(n_cols, XtyCfg::BN);
  return tiles * samples * kTileElems * 2;
}

extern "C" int ghost_persample_tiles_bf16(const void* X, const void* Y, int n_samples_total, long long T, int m_cols,
                                          int n_cols, long long ldx, long long ldy, int sample0, int samples,
                                          int colsum_of, float* colsum_out, void* tiles_out, long long tiles_bytes,
                                          void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(X && Y && tiles_out, "ghost_persample_tiles_bf16: null pointer");
  GB_REQUIRE(colsum_of >= 0 && colsum_of <= 2 && (colsum_of == 0 || colsum_out != nullptr),
             "ghost_persample_tiles_bf16: colsum_of must be 0, 1 (X) or 2 (Y) with an output buffer");
  GB_REQUIRE(T > 0 && T < (1ll << 31) - 64 && m_cols > 0 && n_cols > 0, "ghost_persample_tiles_bf16: bad dimensions");
  GB_REQUIRE(samples > 0 && sample0 >= 0 && sample0 + samples <= n_samples_total,
             "ghost_persample_tiles_bf16: sample range outside the batch");
  GB_REQUIRE(tiles_bytes >= ghost_persample_tiles_bytes(samples, m_cols, n_cols),
             "ghost_persample_tiles_bf16: tile buffer too small");
  GB_REQUIRE((reinterpret_cast<uintptr_t>(tiles_out) & 255u) == 0, "ghost_persample_tiles_bf16: tiles must be 256-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  XtyParams p = {};
  p.mode = kEpiStoreTiles;
  p.m_cols = m_cols;
  p.n_cols = n_cols;
  p.m_tiles = ceil_div(m_cols, XtyCfg::BM);
  p.n_tiles = ceil_div(n_cols, XtyCfg::BN);
  p.T = T;
  p.k_splits = 1;
  p.sample_major = 1;
  p.kb_per_split = ceil_div(T, XtyCfg::BK);
  p.v_is_f32 = 0;
  p.colsum_of = colsum_of;
  p.colsum_out = colsum_out;
  p.cs_src = static_cast<const __nv_bfloat16*>(colsum_of == 1 ? X : Y);
  p.cs_ld = (colsum_of == 1) ? ldx : ldy;
  p.err = ds->err_word;
  p.samples = samples;
  p.sample0 = sample0;
  p.vgrad = tiles_out;
  CUtensorMap tx, ty;
  int rc;
  if ((rc = make_xty_maps(&tx, &ty, p, X, Y, n_samples_total, T, ldx, ldy)) != GHOST_OK) return rc;
  if (pair_kernel_fits(g_persample_pair_mode, m_cols, n_cols) && p.blocked_x && p.blocked_y && xty_pair_usable(ds))
    return launch_xty_pair_tiles(X, Y, n_samples_total, T, m_cols, n_cols, ldx, ldy, samples, sample0, tiles_out, 0,
                                 colsum_of, colsum_out, ds, st);
  return launch_xty(tx, ty, p, ds, st);
}

extern "C" int ghost_tile_dot_bf16(const void* V, int v_ranks, int v_per_rank, const void* W, int n_train, int m_cols,
                                   int n_cols, float dot_scale, float* M_out, void* grad_out, int grad_is_f32,
                                   float grad_scale, int grad_accumulate, void* stream) {
  const DeviceState* ds = device_state();
  if (!ds) return GHOST_ERR_DEVICE;
  GB_REQUIRE(V && W && M_out, "ghost_tile_dot_bf16: null pointer");
  GB_REQUIRE(n_train > 0, "No training samples to compute dot product, check batch sizes.");
  GB_REQUIRE(v_ranks > 0 && v_per_rank > 0 && m_cols > 0 && n_cols > 0, "ghost_tile_dot_bf16: bad dimensions");
  GB_REQUIRE(!grad_out || grad_is_f32 || n_train <= 32,
             "ghost_tile_dot_bf16: a bf16 train gradient is written directly only for up to 32 train samples");
  const int n_val = v_ranks * v_per_rank;
  const int vr = n_val <= 8 ? 8 : (n_val <= 16 ? 16 : 32);
  GB_REQUIRE(vr % v_per_rank == 0 || v_per_rank % vr == 0,
             "ghost_tile_dot_bf16: %d validation samples per rank do not fit the kernel's blocks of %d", v_per_rank, vr);
  GB_REQUIRE((reinterpret_cast<uintptr_t>(V) & 255u) == 0 && (reinterpret_cast<uintptr_t>(W) & 255u) == 0,
             "ghost_tile_dot_bf16: tile buffers must be 256-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n_tiles_n = ceil_div(n_cols, XtyCfg::BN);
  const long long tiles = static_cast<long long>(ceil_div(m_cols, XtyCfg::BM)) * n_tiles_n;
  GB_CUDA_OK(cudaMemsetAsync(M_out, 0, sizeof(float) * static_cast<size_t>(n_val) * n_train, st));
  return launch_tile_dot(V, n_val, 0, W, n_train, 0, tiles, n_val, n_train, 0, n_train, dot_scale, M_out, nullptr, 1,
                         grad_out, grad_is_f32, grad_accumulate, m_cols, n_cols, n_tiles_n, grad_scale, ds, st,
                         v_per_rank);
}
