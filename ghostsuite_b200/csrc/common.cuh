// Host-side plumbing shared by every translation unit of libghost_b200: status codes, the
// thread-local error message, the kernel-launch counter, the per-device error word that kernels
// write when a bounded wait gives up, and TMA tensor-map construction.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/ghost_b200.h"

namespace gb {

// ---- error message (thread local) -------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define GB_CUDA_OK(expr)                                                                   \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess)                                                                 \
      return ::gb::fail(GHOST_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                    \
                        cudaGetErrorString(_e), __FILE__, __LINE__);                       \
  } while (0)

#define GB_REQUIRE(cond, ...)                                                              \
  do {                                                                                     \
    if (!(cond)) return ::gb::fail(GHOST_ERR_INVALID, __VA_ARGS__);                        \
  } while (0)

// ---- launch accounting -------------------------------------------------------------------
void count_launch(int n = 1);
int post_launch(const char* what);  // cudaGetLastError -> status

// Value kernels store in the device error word when they meet an embedding id outside [0, vocab):
// the id's contribution is skipped and ghost_poll_kernel_error reports GHOST_ERR_INDEX.
static constexpr int kErrBadIndex = 9001;

// ---- per-device state ----------------------------------------------------------------------
struct DeviceState {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  int* err_word = nullptr;  // device address of the kernel error word
};
// Returns nullptr (and sets the error) if the current device is not sm_100.
const DeviceState* device_state();

// ---- TMA ---------------------------------------------------------------------------------------
// 2-D row-major bf16 tensor [rows, cols] with row pitch `ld` elements; box = [box_rows, 64 cols]
// (64 bf16 = 128 bytes) with the 128-byte swizzle.  Out-of-bounds elements read as zero.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols = 64);

// 3-D view [samples, rows, cols] of a row-major bf16 matrix (sample pitch = rows * ld); box =
// [1, box_rows, 64 cols].  Rows past the end of a sample read as zero, so a K-loop over one
// sample's tokens never sees its neighbour's.
int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t samples, uint64_t rows,
                      uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols = 64);

// The same matrix seen as [samples, cols/64, rows, 64] (cols a multiple of 64): one box covers
// `box_blocks` adjacent 64-column blocks of `box_rows` rows, each block landing in shared memory
// as its own swizzled [box_rows][64] panel.  Coordinates: (0, row, block, sample).
int make_tmap_bf16_blocks(CUtensorMap* out, const void* base, uint64_t samples, uint64_t rows,
                          uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_blocks);

// Validation tiles as an all-gather leaves them: [ranks][tiles][per_rank samples][32768] bf16, seen as
// [64, per_rank, ranks, 512 panels, tiles]; a box holds `box_rows` consecutive validation samples
// (global index = rank * per_rank + sample) of `box_blocks` panels, each panel a swizzled
// [box_rows][64] block -- the layout make_tmap_bf16_blocks gives for a tile-major buffer.  box_rows
// must divide per_rank or be a multiple of it.  Coordinates: (0, sample, rank, panel, tile).
int make_tmap_bf16_gathered_tiles(CUtensorMap* out, const void* base, uint64_t ranks, uint64_t tiles,
                                  uint64_t per_rank, uint32_t box_rows, uint32_t box_blocks);

// Plain (unswizzled) 2-D map of a row-major matrix of 2- or 4-byte elements; box = [box_rows, box_cols].
int make_tmap_plain_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                       uint64_t ld, uint32_t box_rows, uint32_t box_cols);
// 2-D map of a dense row-major bf16 matrix for tiled STORES of [box_rows, 32 columns] boxes (64-byte
// rows) from shared memory written with the 64-byte swizzle: 16-byte chunk c of row r sits at
// r * 64 + ((c ^ ((r >> 1) & 3)) * 16).
int make_tmap_bf16_store_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);
// Plain 3-D map of a dense [planes, rows, cols] array; box = [1, box_rows, box_cols].
int make_tmap_plain_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t planes, uint64_t rows,
                       uint64_t cols, uint32_t box_rows, uint32_t box_cols);

inline int ceil_div(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

}  // namespace gb
