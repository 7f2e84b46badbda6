// Error string, workspace arena and the device-wide exclusive scan used by the block builder.
#include <stdarg.h>

#include "common.cuh"
#include "scan.cuh"

namespace nb {

static thread_local char g_err[512] = "";
unsigned long long g_launches = 0;

static Tuning g_default_tuning;
static thread_local Tuning *t_tuning = nullptr;
Tuning &default_tuning() { return g_default_tuning; }
Tuning &tuning() { return t_tuning ? *t_tuning : g_default_tuning; }
TuningScope::TuningScope(Tuning *t) : prev(t_tuning) { t_tuning = t; }
TuningScope::~TuningScope() { t_tuning = prev; }

}  // namespace nb

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI passes inter-process handles as 64 bytes");

NB_API int nb_shard_alloc(void **d_ptr, size_t bytes) {
  NB_REQUIRE(d_ptr && bytes > 0, "nb_shard_alloc: null pointer or empty shard");
  NB_CUDA(cudaMalloc(d_ptr, bytes));
  return 0;
}
NB_API int nb_shard_free(void *d_ptr) {
  if (d_ptr) NB_CUDA(cudaFree(d_ptr));
  return 0;
}
NB_API int nb_shard_upload(void *d_dst, const void *src, size_t bytes) {
  NB_REQUIRE(d_dst && src, "nb_shard_upload: null pointer");
  NB_CUDA(cudaMemcpy(d_dst, src, bytes, cudaMemcpyDefault));
  return 0;
}
NB_API int nb_shard_export(void *d_ptr, unsigned char handle[64]) {
  NB_REQUIRE(d_ptr && handle, "nb_shard_export: null pointer");
  cudaIpcMemHandle_t h;
  NB_CUDA(cudaIpcGetMemHandle(&h, d_ptr));
  memcpy(handle, &h, sizeof(h));
  return 0;
}
NB_API int nb_shard_open(const unsigned char handle[64], void **d_ptr) {
  NB_REQUIRE(handle && d_ptr, "nb_shard_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  NB_CUDA(cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
NB_API int nb_shard_close(void *d_ptr) {
  if (d_ptr) NB_CUDA(cudaIpcCloseMemHandle(d_ptr));
  return 0;
}

namespace nb {
cudaError_t wait_stream_host(cudaStream_t stream) {
  if (!tuning().blocking_sync) return cudaStreamSynchronize(stream);
  // one blocking event per thread and device, created on first use and kept for the life of the thread
  thread_local cudaEvent_t ev[kMaxDevices] = {};
  int dev = 0;
  cudaError_t st = cudaGetDevice(&dev);
  if (st != cudaSuccess) return st;
  if (dev < 0 || dev >= kMaxDevices) return cudaStreamSynchronize(stream);
  if (!ev[dev]) {
    st = cudaEventCreateWithFlags(&ev[dev], cudaEventBlockingSync | cudaEventDisableTiming);
    if (st != cudaSuccess) return st;
  }
  st = cudaEventRecord(ev[dev], stream);
  if (st != cudaSuccess) return st;
  return cudaEventSynchronize(ev[dev]);
}

int num_sms() {
  static int cached[kMaxDevices] = {};
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return 148;
  if (cached[d] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) return 148;
    cached[d] = n;
  }
  return cached[d];
}

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

// ---------------------------------------------------------------------------------------------
// Exclusive scan in passes: tile sums -> (scan of the tile sums by one block, for very long inputs) -> per-tile scan.
// No inter-block waiting, so there is nothing that can spin.  Traffic: reads the input twice and
// writes the output once (12 bytes per element for u32 -> u32).
// ---------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void __launch_bounds__(kScanThreads) scan_tile_sums(const uint32_t *__restrict__ in,
                                                               TOut *__restrict__ tile_sums, uint64_t n) {
  __shared__ TOut smem[33];
  uint64_t base = (uint64_t)blockIdx.x * kScanTile;
  TOut sum = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    uint64_t i = base + (uint64_t)k * kScanThreads + threadIdx.x;
    if (i < n) sum += in[i];
  }
  TOut total;
  block_exclusive_scan<TOut>(sum, &total, smem);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

template <typename TOut>
__global__ void __launch_bounds__(1024) scan_tile_offsets(TOut *tile_sums, uint64_t tiles, TOut *grand_total) {
  __shared__ TOut smem[33];
  TOut carry = 0;
  for (uint64_t start = 0; start < tiles; start += 1024) {
    uint64_t i = start + threadIdx.x;
    TOut v = i < tiles ? tile_sums[i] : (TOut)0;
    TOut total;
    TOut ex = block_exclusive_scan<TOut>(v, &total, smem);
    if (i < tiles) tile_sums[i] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0 && grand_total) *grand_total = carry;
}

// Two-pass form for up to kScanThreads * 4 tiles (2 M elements): every block adds up the sums of the tiles
// before its own (at most a thousand values) instead of waiting for a middle launch to scan them.
template <typename TOut>
__global__ void __launch_bounds__(kScanThreads) scan_tiles_self_offset(const uint32_t *in, TOut *out,
                                                                       const TOut *__restrict__ tile_sums, uint64_t n,
                                                                       bool write_total) {
  __shared__ TOut smem[33];
  __shared__ TOut s_offset;
  TOut before = 0;
  for (uint32_t t = threadIdx.x; t < blockIdx.x; t += kScanThreads) before += tile_sums[t];
  TOut off_total;
  block_exclusive_scan<TOut>(before, &off_total, smem);
  if (threadIdx.x == 0) s_offset = off_total;
  __syncthreads();
  uint64_t base = (uint64_t)blockIdx.x * kScanTile + (uint64_t)threadIdx.x * kScanItems;
  uint32_t v[kScanItems];
  TOut sum = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    v[k] = (base + k < n) ? in[base + k] : 0u;
    sum += v[k];
  }
  TOut total;
  TOut ex = block_exclusive_scan<TOut>(sum, &total, smem) + s_offset;
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    if (base + k < n) out[base + k] = ex;
    ex += v[k];
  }
  if (write_total && blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) out[n] = s_offset + total;
}

template <typename TOut>
__global__ void __launch_bounds__(kScanThreads) scan_tiles(const uint32_t *in, TOut *out,
                                                           const TOut *__restrict__ tile_offsets, uint64_t n) {
  __shared__ TOut smem[33];
  uint64_t base = (uint64_t)blockIdx.x * kScanTile + (uint64_t)threadIdx.x * kScanItems;
  uint32_t v[kScanItems];
  TOut sum = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    v[k] = (base + k < n) ? in[base + k] : 0u;
    sum += v[k];
  }
  TOut total;
  TOut ex = block_exclusive_scan<TOut>(sum, &total, smem) + tile_offsets[blockIdx.x];
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    if (base + k < n) out[base + k] = ex;
    ex += v[k];
  }
}

template <typename TOut>
static int scan_impl(nb_ws *ws, const uint32_t *d_in, TOut *d_out, uint64_t n, bool write_total,
                     cudaStream_t stream) {
  if (n == 0) {
    if (write_total) NB_CUDA(cudaMemsetAsync(d_out, 0, sizeof(TOut), stream));
    return 0;
  }
  if (n <= kSingleBlockScanMax) {
    scan_single_block<TOut, ScanLoadArray><<<1, 1024, 0, stream>>>(ScanLoadArray{d_in}, d_out, n, write_total);
    NB_LAUNCH_CHECK();
    return 0;
  }
  NB_REQUIRE(ws != nullptr, "scan: workspace is null");
  WsScope scope(ws);
  uint64_t tiles = (n + kScanTile - 1) / kScanTile;
  TOut *tile_sums = ws->alloc_n<TOut>(tiles);
  if (!tile_sums) return fail(NB_ERR_NOMEM, "scan: workspace arena exhausted");
  scan_tile_sums<TOut><<<(unsigned)tiles, kScanThreads, 0, stream>>>(d_in, tile_sums, n);
  NB_LAUNCH_CHECK();
  if (tiles <= (uint64_t)kScanThreads * 4) {
    scan_tiles_self_offset<TOut><<<(unsigned)tiles, kScanThreads, 0, stream>>>(d_in, d_out, tile_sums, n, write_total);
    NB_LAUNCH_CHECK();
    return 0;
  }
  scan_tile_offsets<TOut><<<1, 1024, 0, stream>>>(tile_sums, tiles, write_total ? d_out + n : nullptr);
  NB_LAUNCH_CHECK();
  scan_tiles<TOut><<<(unsigned)tiles, kScanThreads, 0, stream>>>(d_in, d_out, tile_sums, n);
  NB_LAUNCH_CHECK();
  return 0;
}

int exclusive_scan_u32(nb_ws *ws, const uint32_t *d_in, uint32_t *d_out, uint64_t n, bool write_total,
                       cudaStream_t stream) {
  return scan_impl<uint32_t>(ws, d_in, d_out, n, write_total, stream);
}
int exclusive_scan_u32_to_u64(nb_ws *ws, const uint32_t *d_in, uint64_t *d_out, uint64_t n,
                              bool write_total, cudaStream_t stream) {
  return scan_impl<unsigned long long>(ws, d_in, reinterpret_cast<unsigned long long *>(d_out), n,
                                       write_total, stream);
}

}  // namespace nb

NB_API const char *nb_last_error(void) { return nb::g_err; }
NB_API int nb_version(void) { return 100; }
NB_API uint64_t nb_launch_count(void) { return __atomic_load_n(&nb::g_launches, __ATOMIC_RELAXED); }

NB_API int nb_ws_create(nb_ws **out, void *d_arena, size_t bytes) {
  NB_REQUIRE(out != nullptr, "nb_ws_create: out is null");
  NB_REQUIRE(bytes >= 4096, "nb_ws_create: arena must be at least 4096 bytes");
  nb_ws *ws = new nb_ws();
  if (d_arena) {
    ws->base = static_cast<char *>(d_arena);
    ws->owns = false;
  } else {
    void *p = nullptr;
    cudaError_t err = cudaMalloc(&p, bytes);
    if (err != cudaSuccess) {
      delete ws;
      nb::set_error("nb_ws_create: cudaMalloc(%zu) -> %s", bytes, cudaGetErrorString(err));
      return NB_ERR_CUDA;
    }
    ws->base = static_cast<char *>(p);
    ws->owns = true;
  }
  ws->bytes = bytes;
  cudaError_t err = cudaHostAlloc((void **)&ws->mailbox, 64 * sizeof(uint32_t), cudaHostAllocDefault);
  if (err != cudaSuccess) {
    if (ws->owns) cudaFree(ws->base);
    delete ws;
    nb::set_error("nb_ws_create: cudaHostAlloc -> %s", cudaGetErrorString(err));
    return NB_ERR_CUDA;
  }
  *out = ws;
  return 0;
}

NB_API int nb_ws_destroy(nb_ws *ws) {
  if (!ws) return 0;
  if (ws->mailbox) cudaFreeHost(ws->mailbox);
  if (ws->owns && ws->base) cudaFree(ws->base);
  delete ws;
  return 0;
}

NB_API int nb_ws_reset(nb_ws *ws) {
  NB_REQUIRE(ws != nullptr, "nb_ws_reset: ws is null");
  ws->used = 0;
  return 0;
}
NB_API size_t nb_ws_used(const nb_ws *ws) { return ws ? ws->used : 0; }
NB_API size_t nb_ws_high_water(const nb_ws *ws) { return ws ? ws->high : 0; }
