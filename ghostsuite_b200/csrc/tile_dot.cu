// tile_dot: second half of the per-sample-gradient path.
//
// xty_gemm (kEpiStoreTiles) leaves the per-sample weight-gradient tiles of the validation samples
// (V) and of a group of train samples (W) in a workspace, tile-major: [tile][sample][32768].  V and W
// may be one buffer holding all samples (train first) or two buffers; either way they are described
// by 3-D tensor maps [tiles, samples, 32768] plus a first-validation-sample offset.  This kernel streams both once and produces
//     M[v, b]  += scale * sum_k V[v][k] * W[b][k]        (Frobenius products, reference :135)
//     sum[k]   (+)= sum_b W[b][k]                        (the train gradient, reference :168)
//
// HBM-bound by design, so it is built as a copy pipeline: one producer thread feeds a ring of
// shared-memory stages with TMA (one box of validation rows and one of 32 train rows, 256 elements
// wide, per stage); eight compute warps consume them.  Each CTA owns a contiguous range of stages:
// the train-gradient sum is a plain read-modify-write (deterministic, no atomics); the dot
// products are reduced inside the CTA and added to M once per CTA and block.
//
// bf16 tiles (tile_dot_mma_kernel): the stage is loaded as four 128-byte-swizzled 64-element
// panels per operand, and both contractions run on the tensor cores through mma.sync
// (m16n8k16, fp32 accumulate) fed by ldmatrix: the dot products as W[16 train x 16 k] x
// V[16 k x 8 val], the train-gradient sum as mask[16 x 16 train] x W[16 train x 8 k] (a
// transposed ldmatrix of the same rows).  Warp w owns elements 32w..32w+31 of the stage.  With the
// arithmetic off the CUDA cores the kernel is bound by the stream, and up to 32 validation rows
// share one pass over the train rows.
//
// fp32 tiles (tile_dot_kernel<float>): warp w owns train samples 4w..4w+3 of the block, lane l
// elements 8l..8l+7 of the stage, every shared-memory read is a conflict-free 16-byte access and
// a thread accumulates an 8 x 4 block of dot products on the CUDA cores (exact fp32 products).
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace gb {

constexpr int kTileElems = 128 * 256;
constexpr int kTdCols = 256;            // elements per stage row
constexpr int kTdValRows = 8;
constexpr int kTdTrainRows = 32;

struct TileDotParams {
  long long stages;           // tiles * (32768 / 256)
  long long stages_per_cta;
  int n_val, n_grp;           // validation samples, train samples in this group
  int v_off;                  // index of the first validation sample inside V's sample dimension
  int v_per_rank;             // > 0: V is [ranks][tiles][v_per_rank][32768] (bf16 kernel only), v_off = 0
  int b0, n_train;            // first train sample of the group, total train samples (M row pitch)
  float scale;
  float* M;                   // [n_val, n_train]
  float* sum;                 // [tiles * 32768] fp32 or null
  int sum_init;               // 1: this group overwrites sum, 0: it accumulates
  // direct output of the train gradient (single-group case): out[r, c] (= or +=) out_scale * sum
  void* out;                  // [m_cols, n_cols] row-major in the parameter dtype, or null
  int out_is_f32, out_accumulate;
  int m_cols, n_cols, n_tiles_n;
  float out_scale;
  int* err;
};

template <typename T>
struct TdCfg {
  static constexpr int kRowBytes = kTdCols * sizeof(T);
  static constexpr int kStageBytes = (kTdValRows + kTdTrainRows) * kRowBytes;    // 20 KB / 40 KB
  static constexpr int kStages = sizeof(T) == 2 ? 8 : 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + 8 * kTdCols * 4 + 1024 + 256;
};

__device__ __forceinline__ void td_load8(const __nv_bfloat16* p, float (&x)[8]) {
  const uint4 w = *reinterpret_cast<const uint4*>(p);
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    x[2 * e] = __uint_as_float(ww[e] << 16);
    x[2 * e + 1] = __uint_as_float(ww[e] & 0xffff0000u);
  }
}
__device__ __forceinline__ void td_load8(const float* p, float (&x)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

template <typename T>
__global__ void __launch_bounds__(288, 1)
tile_dot_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_w,
                const TileDotParams p) {
  using Cfg = TdCfg<T>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_part = reinterpret_cast<float*>(smem + kStages * Cfg::kStageBytes);     // [8 warps][256]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes + 8 * kTdCols * 4);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long s_begin = static_cast<long long>(blockIdx.x) * p.stages_per_cta;
  const long long s_end = (s_begin + p.stages_per_cta < p.stages) ? s_begin + p.stages_per_cta : p.stages;
  constexpr int kStagesPerTile = kTileElems / kTdCols;   // 128

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 8); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 8 && lane == 0) { tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_w); }
  __syncthreads();

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int j0 = 0; j0 < p.n_grp && ok; j0 += kTdTrainRows)
        for (int v0 = 0; v0 < p.n_val && ok; v0 += kTdValRows)
          for (long long s = s_begin; s < s_end; ++s) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, 431)) { ok = false; break; }
            uint8_t* st = smem + stage * Cfg::kStageBytes;
            const int tile = static_cast<int>(s / kStagesPerTile);
            const int col = static_cast<int>(s % kStagesPerTile) * kTdCols;
            mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
            tma_load_3d(st, &tm_v, &full_bar[stage], col, p.v_off + v0, tile);
            tma_load_3d(st + kTdValRows * Cfg::kRowBytes, &tm_w, &full_bar[stage], col, j0, tile);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
    }
    return;
  }

  // ------------------------------------------------------------------ compute warps 0-7
  int stage = 0; uint32_t phase = 0;
  bool alive = true;
  for (int j0 = 0; j0 < p.n_grp && alive; j0 += kTdTrainRows) {
    for (int v0 = 0; v0 < p.n_val && alive; v0 += kTdValRows) {
      float acc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[i][q] = 0.f;
      const bool do_sum = (v0 == 0) && (p.sum != nullptr || p.out != nullptr);
      bool bvalid[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) bvalid[q] = (j0 + warp * 4 + q) < p.n_grp;
#pragma unroll 1
      for (long long s = s_begin; s < s_end; ++s) {
        const bool ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.err, 132);
        if (!named_bar_and(1, 256, ok)) { alive = false; break; }
        const T* vbuf = reinterpret_cast<const T*>(smem + stage * Cfg::kStageBytes);
        const T* wbuf = vbuf + kTdValRows * kTdCols;
        float w[4][8];
        float ssum[8];
#pragma unroll
        for (int x = 0; x < 8; ++x) ssum[x] = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          td_load8(wbuf + (warp * 4 + q) * kTdCols + lane * 8, w[q]);
#pragma unroll
          for (int x = 0; x < 8; ++x) ssum[x] += bvalid[q] ? w[q][x] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float vv[8];
          td_load8(vbuf + i * kTdCols + lane * 8, vv);
#pragma unroll
          for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int x = 0; x < 8; ++x) acc[i][q] = fmaf(vv[x], w[q][x], acc[i][q]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);     // this warp is done with the stage
        if (++stage == kStages) { stage = 0; phase ^= 1; }
        if (do_sum) {
          float4* mine = reinterpret_cast<float4*>(s_part + warp * kTdCols + lane * 8);
          mine[0] = make_float4(ssum[0], ssum[1], ssum[2], ssum[3]);
          mine[1] = make_float4(ssum[4], ssum[5], ssum[6], ssum[7]);
          asm volatile("bar.sync 2, 256;" ::: "memory");
          float t = 0.f;
#pragma unroll
          for (int ww = 0; ww < 8; ++ww) t += s_part[ww * kTdCols + threadIdx.x];
          if (p.out != nullptr) {
            // one stage is one 256-column row segment of one 128 x 256 tile
            const long long tile = s / kStagesPerTile;
            const int r = static_cast<int>(tile / p.n_tiles_n) * 128 + static_cast<int>(s % kStagesPerTile);
            const int c = static_cast<int>(tile % p.n_tiles_n) * 256 + static_cast<int>(threadIdx.x);
            if (r < p.m_cols && c < p.n_cols) {
              const long long o = static_cast<long long>(r) * p.n_cols + c;
              float val = t * p.out_scale;
              if (p.out_is_f32) {
                float* dst = static_cast<float*>(p.out) + o;
                if (p.out_accumulate || j0 > 0) val += *dst;
                *dst = val;
              } else {
                __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + o;
                if (p.out_accumulate || j0 > 0) val += __bfloat162float(*dst);
                *dst = __float2bfloat16_rn(val);
              }
            }
          } else {
            float* dst = p.sum + s * kTdCols + threadIdx.x;
            if (!(p.sum_init && j0 == 0)) t += *dst;
            *dst = t;
          }
        }
      }
      if (!alive) break;
      // reduce the 8 x 4 block over the 32 lanes, one atomic per (v, b) and CTA
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float a = acc[i][q];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
          const int v = v0 + i, b = j0 + warp * 4 + q;
          if (lane == 0 && v < p.n_val && b < p.n_grp && a != 0.f)
            atomicAdd(&p.M[static_cast<long long>(v) * p.n_train + p.b0 + b], a * p.scale);
        }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// bf16 tiles on mma.sync
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Elements per stage row of the bf16 kernel.  Every warp pays a barrier wait per stage, so a stage
// is made as wide as the shared memory allows: 512 elements = 64 per warp = four k-steps.
constexpr int kMmaCols = 512;

// NVT: 8-row validation blocks per stage (1, 2 or 4); MT: 16-row train blocks per stage (2, or 1
// when the group has at most 16 train samples: a data-parallel rank's share of the batch -- the
// stage then holds and the warps then work on half as many rows)
template <int NVT, int MT = 2>
struct TdMmaCfg {
  static constexpr int kTrainRows = 16 * MT;
  static constexpr int kValRows = 8 * NVT;
  static constexpr int kPanels = kMmaCols / 64;                              // 64-element panels per stage row
  static constexpr int kWarpChunks = kMmaCols / 8 / 8;                       // 16-byte chunks per warp and stage
  static constexpr int kWarpKSteps = kWarpChunks / 2;
  static constexpr int kValBytes = kPanels * kValRows * 128;
  static constexpr int kStageBytes = kValBytes + kPanels * kTrainRows * 128;     // 40 / 48 / 64 KB at MT = 2
  static constexpr int kStages = NVT == 1 ? 4 : 3;
  static constexpr int kRedBytes = 8 * kTrainRows * kValRows * 4;            // per-warp partial dot blocks
  static constexpr int kSmemBytes = kStages * kStageBytes + kRedBytes + 1024 + 256;
};

template <int NVT, int MT>
__global__ void __launch_bounds__(288, 1)
tile_dot_mma_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_w,
                    const TileDotParams p) {
  using Cfg = TdMmaCfg<NVT, MT>;
  constexpr int kStages = Cfg::kStages, VR = Cfg::kValRows, TR = Cfg::kTrainRows;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_red = reinterpret_cast<float*>(smem + kStages * Cfg::kStageBytes);            // [8 warps][32][VR]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes + Cfg::kRedBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long s_begin = static_cast<long long>(blockIdx.x) * p.stages_per_cta;
  const long long s_end = (s_begin + p.stages_per_cta < p.stages) ? s_begin + p.stages_per_cta : p.stages;
  constexpr int kStagesPerTile = kTileElems / kMmaCols;   // 64
  constexpr int KS = Cfg::kWarpKSteps, CW = Cfg::kWarpChunks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 8); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 8 && lane == 0) { tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_w); }
  __syncthreads();

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int j0 = 0; j0 < p.n_grp && ok; j0 += TR)
        for (int v0 = 0; v0 < p.n_val && ok; v0 += VR)
          for (long long s = s_begin; s < s_end; ++s) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, 431)) { ok = false; break; }
            uint8_t* st = smem + stage * Cfg::kStageBytes;
            const int tile = static_cast<int>(s / kStagesPerTile);
            const int panel = static_cast<int>(s % kStagesPerTile) * Cfg::kPanels;   // 64-element panels
            mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
            if (p.v_per_rank > 0)
              tma_load_5d(st, &tm_v, &full_bar[stage], 0, v0 % p.v_per_rank, v0 / p.v_per_rank, panel, tile);
            else
              tma_load_4d(st, &tm_v, &full_bar[stage], 0, p.v_off + v0, panel, tile);
            tma_load_4d(st + Cfg::kValBytes, &tm_w, &full_bar[stage], 0, j0, panel, tile);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
    }
    return;
  }

  // ------------------------------------------------------------------ compute warps 0-7
  // This warp's slice of a stage: CW 16-byte chunks (KS k-steps) starting at chunk c0 of panel pn.
  const int pn = (warp * CW) / 8, c0 = (warp * CW) % 8;
  const int g = lane >> 2, q = lane & 3;
  // ldmatrix lane addresses inside a stage (panel rows are 128 bytes, chunk index XOR (row & 7))
  uint32_t a_off[MT][KS];    // W as the A operand: [m-tile][k-step]
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int row = mt * 16 + (lane & 15), chunk = c0 + 2 * ks + (lane >> 4);
      a_off[mt][ks] = Cfg::kValBytes + pn * (TR * 128) + row * 128 + ((chunk ^ (row & 7)) << 4);
    }
  uint32_t b_off[NVT][KS / 2];   // V as the B operand: [n-tile][pair of k-steps], one x4 each
#pragma unroll
  for (int nt = 0; nt < NVT; ++nt)
#pragma unroll
    for (int h = 0; h < KS / 2; ++h) {
      const int row = nt * 8 + (lane & 7), chunk = c0 + 4 * h + (lane >> 3);
      b_off[nt][h] = pn * (VR * 128) + row * 128 + ((chunk ^ (row & 7)) << 4);
    }
  uint32_t t_off[CW];        // W transposed, for the column sums: [8-element group], rows = lane
  const int trow = lane & (TR - 1);      // with 16 train rows lanes 16-31 repeat rows 0-15 (their matrices are not used)
#pragma unroll
  for (int j = 0; j < CW; ++j)
    t_off[j] = Cfg::kValBytes + pn * (TR * 128) + trow * 128 + (((c0 + j) ^ (trow & 7)) << 4);

  int stage = 0; uint32_t phase = 0;
  bool alive = true;
  for (int j0 = 0; j0 < p.n_grp && alive; j0 += TR) {
    // A operand of the column-sum MMA: 1.0 where the train row (the k index) belongs to the group
    uint32_t mask_a[2][4];
#pragma unroll
    for (int kr = 0; kr < 2; ++kr) {
      const int k_lo = j0 + kr * 16 + q * 2, k_hi = k_lo + 8;
      const uint32_t lo = (k_lo < p.n_grp ? 0x3F80u : 0u) | (k_lo + 1 < p.n_grp ? 0x3F800000u : 0u);
      const uint32_t hi = (k_hi < p.n_grp ? 0x3F80u : 0u) | (k_hi + 1 < p.n_grp ? 0x3F800000u : 0u);
      mask_a[kr][0] = lo; mask_a[kr][1] = lo; mask_a[kr][2] = hi; mask_a[kr][3] = hi;
    }
    for (int v0 = 0; v0 < p.n_val && alive; v0 += VR) {
      float acc[MT][NVT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NVT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[mt][nt][e] = 0.f;
      const bool do_sum = (v0 == 0) && (p.sum != nullptr || p.out != nullptr);
#pragma unroll 1
      for (long long s = s_begin; s < s_end; ++s) {
        // the warps run through the ring independently of one another; lane 0 waits for the warp
        int ok = 1;
        if (lane == 0) ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.err, 132) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { alive = false; break; }
        const uint32_t st = smem_u32(smem + stage * Cfg::kStageBytes);
        uint32_t a[MT][KS][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) ldsm_x4(st + a_off[mt][ks], a[mt][ks]);
#pragma unroll
        for (int nt = 0; nt < NVT; ++nt)
#pragma unroll
          for (int h = 0; h < KS / 2; ++h) {
            uint32_t b[4];
            ldsm_x4(st + b_off[nt][h], b);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_bf16_16816(acc[mt][nt], a[mt][2 * h], b[0], b[1]);
              mma_bf16_16816(acc[mt][nt], a[mt][2 * h + 1], b[2], b[3]);
            }
          }
        float t0 = 0.f, t1 = 0.f;
        if (do_sum) {
          // every row of the column-sum accumulator holds the sums of 8 elements of this warp's
          // slice; lane (g, q) keeps elements 8g + 2q, 8g + 2q + 1 of each group of 64
#pragma unroll
          for (int j = 0; j < CW; ++j) {
            uint32_t t[4];
            float cs[4] = {0.f, 0.f, 0.f, 0.f};
            ldsm_x4_trans(st + t_off[j], t);
            mma_bf16_16816(cs, mask_a[0], t[0], t[1]);
            if (MT == 2) mma_bf16_16816(cs, mask_a[1], t[2], t[3]);
            if (g == (j & 7)) { t0 = cs[0]; t1 = cs[1]; }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);     // this warp is done with the stage
        if (++stage == kStages) { stage = 0; phase ^= 1; }
        if (do_sum && g < CW) {
          const int e0 = warp * (CW * 8) + g * 8 + q * 2;    // element inside the stage
          if (p.out != nullptr) {
            // one stage is kMmaCols / 256 row segments (256 columns each) of one 128 x 256 tile
            const long long tile = s / kStagesPerTile;
            const int r = static_cast<int>(tile / p.n_tiles_n) * 128 +
                          static_cast<int>(s % kStagesPerTile) * (kMmaCols / 256) + (e0 >> 8);
            const int c = static_cast<int>(tile % p.n_tiles_n) * 256 + (e0 & 255);
            if (r < p.m_cols && c < p.n_cols) {
              const long long o = static_cast<long long>(r) * p.n_cols + c;
              const bool rmw = p.out_accumulate || j0 > 0;
              const bool pair = (c + 1 < p.n_cols) && ((p.n_cols & 1) == 0);     // o is even then
              t0 *= p.out_scale; t1 *= p.out_scale;
              if (p.out_is_f32) {
                float* dst = static_cast<float*>(p.out) + o;
                if (pair) {
                  float2 v = make_float2(t0, t1);
                  if (rmw) { const float2 old = *reinterpret_cast<const float2*>(dst); v.x += old.x; v.y += old.y; }
                  *reinterpret_cast<float2*>(dst) = v;
                } else {
                  dst[0] = rmw ? dst[0] + t0 : t0;
                  if (c + 1 < p.n_cols) dst[1] = rmw ? dst[1] + t1 : t1;
                }
              } else {
                __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + o;
                if (pair) {
                  if (rmw) {
                    const __nv_bfloat162 old = *reinterpret_cast<const __nv_bfloat162*>(dst);
                    t0 += __bfloat162float(old.x); t1 += __bfloat162float(old.y);
                  }
                  *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(t0, t1);
                } else {
                  dst[0] = __float2bfloat16_rn(rmw ? __bfloat162float(dst[0]) + t0 : t0);
                  if (c + 1 < p.n_cols) dst[1] = __float2bfloat16_rn(rmw ? __bfloat162float(dst[1]) + t1 : t1);
                }
              }
            }
          } else {
            float2* dst = reinterpret_cast<float2*>(p.sum + s * kMmaCols + e0);
            float2 v = make_float2(t0, t1);
            if (!(p.sum_init && j0 == 0)) { const float2 old = *dst; v.x += old.x; v.y += old.y; }
            *dst = v;
          }
        }
      }
      // the only CTA-wide agreement: every compute warp gets here once per block, aborted or not
      if (!named_bar_and(1, 256, alive)) { alive = false; break; }
      // reduce the per-warp [32 train x VR val] partial blocks, one atomic per (v, b) and CTA
      float* mine = s_red + warp * (TR * VR);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NVT; ++nt) {
          const int b_lo = mt * 16 + g, v = nt * 8 + q * 2;
          mine[b_lo * VR + v] = acc[mt][nt][0];
          mine[b_lo * VR + v + 1] = acc[mt][nt][1];
          mine[(b_lo + 8) * VR + v] = acc[mt][nt][2];
          mine[(b_lo + 8) * VR + v + 1] = acc[mt][nt][3];
        }
      asm volatile("bar.sync 2, 256;" ::: "memory");
      for (int idx = threadIdx.x; idx < TR * VR; idx += 256) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += s_red[w * (TR * VR) + idx];
        const int b = j0 + idx / VR, v = v0 + idx % VR;
        if (v < p.n_val && b < p.n_grp && t != 0.f)
          atomicAdd(&p.M[static_cast<long long>(v) * p.n_train + p.b0 + b], t * p.scale);
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");
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

template <typename T>
static int launch_tile_dot_t(const void* V, int v_samples, const void* W, int w_samples, long long tiles,
                             TileDotParams& p, const DeviceState* ds, cudaStream_t st) {
  using Cfg = TdCfg<T>;
  CUtensorMap tv, tw;
  int rc;
  if ((rc = make_tmap_plain_3d(&tv, V, sizeof(T), tiles, v_samples, kTileElems, kTdValRows, kTdCols)) != GHOST_OK)
    return rc;
  if ((rc = make_tmap_plain_3d(&tw, W, sizeof(T), tiles, w_samples, kTileElems, kTdTrainRows, kTdCols)) != GHOST_OK)
    return rc;
  static bool attr_set[64] = {};
  if (!attr_set[ds->device]) {
    GB_CUDA_OK(cudaFuncSetAttribute(tile_dot_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set[ds->device] = true;
  }
  long long ctas = ds->sm_count;
  if (ctas > p.stages) ctas = p.stages;
  p.stages_per_cta = (p.stages + ctas - 1) / ctas;
  ctas = (p.stages + p.stages_per_cta - 1) / p.stages_per_cta;
  tile_dot_kernel<T><<<static_cast<int>(ctas), 288, Cfg::kSmemBytes, st>>>(tv, tw, p);
  count_launch();
  return post_launch("tile_dot_kernel");
}

template <int NVT, int MT>
static int launch_tile_dot_mma_t(const void* V, int v_samples, const void* W, int w_samples, long long tiles,
                                 TileDotParams& p, const DeviceState* ds, cudaStream_t st) {
  using Cfg = TdMmaCfg<NVT, MT>;
  CUtensorMap tv, tw;
  int rc;
  // [tiles][samples][32768] seen as [tiles][512 panels][samples][64]: one box = 4 panels of the stage
  if (p.v_per_rank > 0)
    rc = make_tmap_bf16_gathered_tiles(&tv, V, v_samples / p.v_per_rank, tiles, p.v_per_rank, Cfg::kValRows, Cfg::kPanels);
  else
    rc = make_tmap_bf16_blocks(&tv, V, tiles, v_samples, kTileElems, kTileElems, Cfg::kValRows, Cfg::kPanels);
  if (rc != GHOST_OK) return rc;
  if ((rc = make_tmap_bf16_blocks(&tw, W, tiles, w_samples, kTileElems, kTileElems, Cfg::kTrainRows, Cfg::kPanels)) != GHOST_OK)
    return rc;
  static bool attr_set[64] = {};
  if (!attr_set[ds->device]) {
    GB_CUDA_OK(cudaFuncSetAttribute(tile_dot_mma_kernel<NVT, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set[ds->device] = true;
  }
  long long ctas = ds->sm_count;
  if (ctas > p.stages) ctas = p.stages;
  p.stages_per_cta = (p.stages + ctas - 1) / ctas;
  ctas = (p.stages + p.stages_per_cta - 1) / p.stages_per_cta;
  tile_dot_mma_kernel<NVT, MT><<<static_cast<int>(ctas), 288, Cfg::kSmemBytes, st>>>(tv, tw, p);
  count_launch();
  return post_launch("tile_dot_mma_kernel");
}

template <int NVT>
static int launch_tile_dot_mma(const void* V, int v_samples, const void* W, int w_samples, long long tiles,
                               TileDotParams& p, const DeviceState* ds, cudaStream_t st) {
  if (p.n_grp <= 16) return launch_tile_dot_mma_t<NVT, 1>(V, v_samples, W, w_samples, tiles, p, ds, st);
  return launch_tile_dot_mma_t<NVT, 2>(V, v_samples, W, w_samples, tiles, p, ds, st);
}

// V: [tiles][v_samples][32768] with the validation samples at index v_off..v_off+n_val-1;
// W: [tiles][w_samples][32768] with the group's train samples at index 0..n_grp-1.
// v_per_rank > 0: V holds validation samples only, as an all-gather over ranks leaves them,
// [v_samples / v_per_rank ranks][tiles][v_per_rank][32768] (bf16).
int launch_tile_dot(const void* V, int v_samples, int v_off, const void* W, int w_samples, int is_f32,
                    long long tiles, int n_val, int n_grp, int b0, int n_train, float scale, float* M,
                    float* sum, int sum_init, void* out, int out_is_f32, int out_accumulate, int m_cols,
                    int n_cols, int n_tiles_n, float out_scale, const DeviceState* ds, cudaStream_t st,
                    int v_per_rank) {
  TileDotParams p;
  p.v_off = v_off;
  p.v_per_rank = v_per_rank;
  p.out = out; p.out_is_f32 = out_is_f32; p.out_accumulate = out_accumulate;
  p.m_cols = m_cols; p.n_cols = n_cols; p.n_tiles_n = n_tiles_n; p.out_scale = out_scale;
  p.stages = tiles * (kTileElems / (is_f32 ? kTdCols : kMmaCols));
  p.stages_per_cta = 0;
  p.n_val = n_val; p.n_grp = n_grp; p.b0 = b0; p.n_train = n_train;
  p.scale = scale; p.M = M; p.sum = sum; p.sum_init = sum_init;
  p.err = ds->err_word;
  if (is_f32) return launch_tile_dot_t<float>(V, v_samples, W, w_samples, tiles, p, ds, st);
  if (n_val <= 8) return launch_tile_dot_mma<1>(V, v_samples, W, w_samples, tiles, p, ds, st);
  if (n_val <= 16) return launch_tile_dot_mma<2>(V, v_samples, W, w_samples, tiles, p, ds, st);
  return launch_tile_dot_mma<4>(V, v_samples, W, w_samples, tiles, p, ds, st);
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
