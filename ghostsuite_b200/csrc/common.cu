#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace gb {

static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int post_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GHOST_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return GHOST_OK;
}

// The error word kernels write to.  One copy per device that loads the library.
__device__ int g_kernel_error_word;

static std::mutex g_state_mu;
static DeviceState g_states[64];

const DeviceState* device_state() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("no current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_state_mu);
  DeviceState& s = g_states[dev];
  if (s.device == dev) return &s;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
    set_error("cudaGetDeviceProperties failed");
    return nullptr;
  }
  if (prop.major != 10) {
    set_error("libghost_b200 needs an sm_100 (B200) device, found sm_%d%d", prop.major, prop.minor);
    return nullptr;
  }
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_kernel_error_word) != cudaSuccess) {
    set_error("cudaGetSymbolAddress(error word) failed");
    return nullptr;
  }
  int zero = 0;
  if (cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) {
    set_error("could not clear the device error word");
    return nullptr;
  }
  s.sm_count = prop.multiProcessorCount;
  s.cc_major = prop.major;
  s.cc_minor = prop.minor;
  s.err_word = static_cast<int*>(p);
  s.device = dev;
  return &s;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(GHOST_ERR_INVALID, "TMA operand base %p is not 16-byte aligned", base);
  if ((ld * 2) % 16 != 0)
    return fail(GHOST_ERR_INVALID, "TMA operand row pitch %llu elements is not a multiple of 8",
                (unsigned long long)ld);
  if (rows == 0 || cols == 0) return fail(GHOST_ERR_INVALID, "empty TMA operand");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu cols=%llu ld=%llu)",
                (int)r, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld);
  return GHOST_OK;
}

int make_tmap_plain_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                       uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (ld * elem_bytes) % 16 != 0)
    return fail(GHOST_ERR_INVALID, "TMA operand %p / pitch %llu is not 16-byte aligned", base,
                (unsigned long long)ld);
  if (rows == 0 || cols == 0 || box_cols > 256 || box_rows > 256)
    return fail(GHOST_ERR_INVALID, "bad plain TMA map (rows=%llu cols=%llu box=%ux%u)",
                (unsigned long long)rows, (unsigned long long)cols, box_rows, box_cols);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                  2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled(plain) failed with CUresult %d", (int)r);
  return GHOST_OK;
}

int make_tmap_bf16_store_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || cols % 32 != 0)
    return fail(GHOST_ERR_INVALID, "TMA store target %p / %llu columns: needs 16-byte alignment and a multiple of 32 columns",
                base, (unsigned long long)cols);
  if (rows == 0 || rows >= (1ull << 32) || box_rows == 0 || box_rows > 256)
    return fail(GHOST_ERR_INVALID, "bad TMA store map (rows=%llu box_rows=%u)", (unsigned long long)rows, box_rows);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {32, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled(store) failed with CUresult %d", (int)r);
  return GHOST_OK;
}

int make_tmap_plain_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t planes, uint64_t rows,
                       uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (cols * elem_bytes) % 16 != 0)
    return fail(GHOST_ERR_INVALID, "TMA operand %p / row of %llu elements is not 16-byte aligned", base,
                (unsigned long long)cols);
  if (planes == 0 || rows == 0 || cols == 0 || box_cols > 256 || box_rows > 256)
    return fail(GHOST_ERR_INVALID, "bad plain 3-D TMA map");
  cuuint64_t dims[3] = {cols, rows, planes};
  cuuint64_t strides[2] = {cols * elem_bytes, rows * cols * elem_bytes};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                  3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled(plain 3d) failed with CUresult %d", (int)r);
  return GHOST_OK;
}

int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t samples, uint64_t rows,
                      uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(GHOST_ERR_INVALID, "TMA operand base %p is not 16-byte aligned", base);
  if ((ld * 2) % 16 != 0)
    return fail(GHOST_ERR_INVALID, "TMA operand row pitch %llu elements is not a multiple of 8",
                (unsigned long long)ld);
  if (rows == 0 || cols == 0 || samples == 0) return fail(GHOST_ERR_INVALID, "empty TMA operand");
  cuuint64_t dims[3] = {cols, rows, samples};
  cuuint64_t strides[2] = {ld * 2, rows * ld * 2};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled(3d) failed with CUresult %d", (int)r);
  return GHOST_OK;
}

// [samples, rows, cols] bf16 seen as [samples, cols/64, rows, 64]: one box then covers `box_blocks`
// adjacent 64-column blocks of `box_rows` rows, each block landing in shared memory as its own
// 128-byte-swizzled [box_rows][64] panel.  cols must be a multiple of 64 (a partial last block
// would read past the row instead of being zero-filled).
int make_tmap_bf16_blocks(CUtensorMap* out, const void* base, uint64_t samples, uint64_t rows,
                          uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_blocks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(GHOST_ERR_INVALID, "TMA operand base %p is not 16-byte aligned", base);
  if ((ld * 2) % 16 != 0)
    return fail(GHOST_ERR_INVALID, "TMA operand row pitch %llu elements is not a multiple of 8",
                (unsigned long long)ld);
  if (rows == 0 || cols == 0 || samples == 0 || cols % 64 != 0)
    return fail(GHOST_ERR_INVALID, "blocked TMA operand needs a column count that is a multiple of 64");
  cuuint64_t dims[4] = {64, rows, cols / 64, samples};
  cuuint64_t strides[3] = {ld * 2, 128, rows * ld * 2};
  cuuint32_t box[4] = {64, box_rows, box_blocks, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled(blocked 4d) failed with CUresult %d", (int)r);
  return GHOST_OK;
}

int make_tmap_bf16_gathered_tiles(CUtensorMap* out, const void* base, uint64_t ranks, uint64_t tiles,
                                  uint64_t per_rank, uint32_t box_rows, uint32_t box_blocks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(GHOST_ERR_INVALID, "TMA operand base %p is not 16-byte aligned", base);
  if (ranks == 0 || tiles == 0 || per_rank == 0 || box_rows == 0 ||
      !(box_rows % per_rank == 0 || per_rank % box_rows == 0))
    return fail(GHOST_ERR_INVALID, "gathered tiles: %llu samples per rank do not fit boxes of %u rows",
                (unsigned long long)per_rank, box_rows);
  const uint64_t tile_bytes = 32768ull * 2;
  const uint32_t bs = box_rows < per_rank ? box_rows : static_cast<uint32_t>(per_rank);
  cuuint64_t dims[5] = {64, per_rank, ranks, 512, tiles};
  cuuint64_t strides[4] = {tile_bytes, tiles * per_rank * tile_bytes, 128, per_rank * tile_bytes};
  cuuint32_t box[5] = {64, bs, box_rows / bs, box_blocks, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(GHOST_ERR_CUDA, "cuTensorMapEncodeTiled(gathered tiles) failed with CUresult %d", (int)r);
  return GHOST_OK;
}

}  // namespace gb

extern "C" {

const char* ghost_last_error(void) { return gb::g_err; }
const char* ghost_version(void) { return "ghost_b200 0.1 (sm_100a)"; }
long long ghost_launch_count(void) { return gb::g_launches.load(); }

int ghost_device_check(void) { return gb::device_state() ? GHOST_OK : GHOST_ERR_DEVICE; }

int ghost_sm_count(void) {
  const gb::DeviceState* s = gb::device_state();
  return s ? s->sm_count : GHOST_ERR_DEVICE;
}

int ghost_poll_kernel_error(int clear) {
  const gb::DeviceState* s = gb::device_state();
  if (!s) return GHOST_ERR_DEVICE;
  int v = 0;
  if (cudaMemcpy(&v, s->err_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return gb::fail(GHOST_ERR_CUDA, "reading the kernel error word failed: %s",
                    cudaGetErrorString(cudaGetLastError()));
  if (v != 0) {
    if (clear) {
      int zero = 0;
      cudaMemcpy(s->err_word, &zero, sizeof(int), cudaMemcpyHostToDevice);
    }
    if (v == gb::kErrBadIndex) {
      gb::set_error("an embedding id outside [0, vocab) reached a kernel (its contribution was skipped)");
      return GHOST_ERR_INDEX;
    }
    gb::set_error("a kernel gave up a bounded wait (code %d: role %d, barrier kind %d)", v, v / 100,
                  v % 100);
    return GHOST_ERR_KERNEL_TIMEOUT;
  }
  return GHOST_OK;
}

}  // extern "C"
