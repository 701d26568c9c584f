// Device context, refcounted storage with a caching allocator, host<->device transfers.
//
// Stands in for the reference's WebGPUDeviceManager / WebGPUStorage pair
// (packages/backend-webgpu/src/base/device.ts:95-176, base/storage.ts:60-243): storages are
// refcounted, views share a storage, release at refcount 0 returns the block to a free list.
// Everything is ordered on one stream, so a block can be reused as soon as it is released.
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "kernels.cuh"

namespace kd {

static thread_local std::string g_last_error;

void set_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
}

int fail(int status, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return status;
}

static Context g_ctx;
Context& ctx() { return g_ctx; }

int require_init() {
  if (!g_ctx.ready) return fail(KD_ERR_NOT_INIT, "kd_init has not been called");
  return KD_OK;
}

int after_launch(const char* name) {
  g_ctx.launches++;
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(KD_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e));
  }
  return KD_OK;
}

// ----------------------------------------------------------------------------- allocator
struct Allocator {
  std::mutex mu;
  std::multimap<uint64_t, void*> free_blocks;  // block size -> ptr
  std::unordered_map<uint64_t, Storage*> live; // handle -> storage
  uint64_t next_handle = 1;
  uint64_t in_use = 0, cached = 0, reserved = 0;

  static uint64_t round_size(uint64_t bytes) {
    if (bytes == 0) bytes = 1;
    if (bytes <= (1u << 20)) return (bytes + 511) & ~uint64_t(511);
    const uint64_t g = 2u << 20;  // 2 MiB granularity for large blocks
    return (bytes + g - 1) / g * g;
  }

  int alloc_block(uint64_t block, void** out, uint64_t* actual) {
    *actual = block;
    auto it = free_blocks.lower_bound(block);
    // Reuse a cached block when it wastes at most 25 %.
    if (it != free_blocks.end() && it->first <= block + block / 4) {
      *out = it->second;
      *actual = it->first;
      cached -= it->first;
      in_use += it->first;
      free_blocks.erase(it);
      return KD_OK;
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, block);
    if (e != cudaSuccess) {
      cudaGetLastError();
      release_cached();
      e = cudaMalloc(&p, block);
    }
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(KD_ERR_OOM, "device allocation of %llu bytes failed: %s",
                  (unsigned long long)block, cudaGetErrorString(e));
    }
    reserved += block;
    in_use += block;
    *out = p;
    return KD_OK;
  }

  void release_cached() {
    for (auto& kv : free_blocks) {
      cudaFree(kv.second);
      reserved -= kv.first;
      cached -= kv.first;
    }
    free_blocks.clear();
  }
};

static Allocator g_alloc;

int storage_lookup(uint64_t handle, Storage** out) {
  std::lock_guard<std::mutex> lk(g_alloc.mu);
  auto it = g_alloc.live.find(handle);
  if (it == g_alloc.live.end()) return fail(KD_ERR_INVALID, "unknown or released storage handle %llu",
                                            (unsigned long long)handle);
  *out = it->second;
  return KD_OK;
}

int tensor_ptr(const kd_tensor* t, void** out) {
  if (t == nullptr) return fail(KD_ERR_INVALID, "null tensor");
  if (t->ndim < 0 || t->ndim > KD_MAX_DIMS) return fail(KD_ERR_INVALID, "tensor rank %d out of range", t->ndim);
  Storage* s = nullptr;
  KD_TRY(storage_lookup(t->storage, &s));
  // Bounds: the furthest element addressed by the view must lie inside the storage.
  int64_t lo = t->offset, hi = t->offset;
  bool empty = false;
  for (int i = 0; i < t->ndim; ++i) {
    if (t->shape[i] < 0) return fail(KD_ERR_INVALID, "negative extent");
    if (t->shape[i] == 0) empty = true;
    const int64_t span = (t->shape[i] - 1) * t->strides[i];
    if (span >= 0) hi += span; else lo += span;
  }
  const int esz = dtype_size(t->dtype);
  if (!empty && (lo < 0 || (uint64_t)(hi + 1) * esz > s->bytes))
    return fail(KD_ERR_INVALID, "tensor view [%lld,%lld] elements exceeds its storage of %llu bytes",
                (long long)lo, (long long)hi, (unsigned long long)s->bytes);
  *out = static_cast<char*>(s->ptr) + t->offset * esz;
  return KD_OK;
}

// Scratch buffers that were outgrown.  They are kept until kd_shutdown instead of being freed at
// once: a captured CUDA graph may still hold their address (decode attention
// partial sums, chain partial sums, sampling probabilities), and kernels already enqueued may
// still use them.  Sizes grow by 1.5x, so the retired buffers sum to less than three times the last.
static std::vector<void*> g_retired_workspaces;

int get_workspace(uint64_t bytes, void** out) {
  Context& c = ctx();
  if (bytes > c.workspace_bytes) {
    const uint64_t want = Allocator::round_size(bytes + bytes / 2);
    void* fresh = nullptr;
    cudaError_t e = cudaMalloc(&fresh, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(KD_ERR_OOM, "workspace allocation of %llu bytes failed", (unsigned long long)want);
    }
    if (c.workspace) g_retired_workspaces.push_back(c.workspace);
    c.workspace = fresh;
    c.workspace_bytes = want;
  }
  *out = c.workspace;
  return KD_OK;
}

// Frees the outgrown scratch buffers (shutdown only: no graph built before can run afterwards).
static void release_retired_workspaces() {
  for (void* p : g_retired_workspaces) cudaFree(p);
  g_retired_workspaces.clear();
}

}  // namespace kd

namespace kd { int decode_chain_reset_counters(); int decode_layer_reset_counters(); int p2p_shutdown(); }

using namespace kd;

KD_API int kd_device_count(int* count) {
  if (!count) return fail(KD_ERR_INVALID, "null argument");
  cudaError_t e = cudaGetDeviceCount(count);
  if (e != cudaSuccess) {
    cudaGetLastError();
    *count = 0;
    return fail(KD_ERR_CUDA, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
  }
  return KD_OK;
}

KD_API int kd_init(int device_ordinal, unsigned flags) {
  (void)flags;
  Context& c = ctx();
  if (c.ready) {
    if (c.device == device_ordinal) return KD_OK;
    // launch state (tensor maps, counters, scratch) is kept per process for ONE device: a second
    // device needs kd_shutdown first, or a process of its own (one process drives one GPU)
    return fail(KD_ERR_UNSUPPORTED, "already initialised on device %d: one process drives one GPU (kd_shutdown first)", c.device);
  }
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    cudaGetLastError();
    return fail(KD_ERR_CUDA, "no CUDA device available (%s); this backend has no CPU fallback",
                e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
  }
  KD_REQUIRE(device_ordinal >= 0 && device_ordinal < n, "device ordinal %d out of range (0..%d)", device_ordinal, n - 1);
  KD_CUDA_CHECK(cudaSetDevice(device_ordinal));
  cudaDeviceProp prop;
  KD_CUDA_CHECK(cudaGetDeviceProperties(&prop, device_ordinal));
  if (prop.major != 10)
    return fail(KD_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device_ordinal,
                prop.major, prop.minor);
  c.device = device_ordinal;
  c.sm_count = prop.multiProcessorCount;
  KD_CUDA_CHECK(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
  KD_CUDA_CHECK(cudaMalloc(&c.error_flag, sizeof(int) * 4));
  KD_CUDA_CHECK(cudaMemsetAsync(c.error_flag, 0, sizeof(int) * 4, c.stream));
  c.launches = 0;
  c.ready = true;
  return KD_OK;
}

KD_API int kd_shutdown(void) {
  Context& c = ctx();
  if (!c.ready) return KD_OK;
  cudaStreamSynchronize(c.stream);
  p2p_shutdown();
  {
    std::lock_guard<std::mutex> lk(g_alloc.mu);
    for (auto& kv : g_alloc.live) {
      cudaFree(kv.second->ptr);
      delete kv.second;
    }
    g_alloc.live.clear();
    g_alloc.release_cached();
    g_alloc.in_use = g_alloc.cached = g_alloc.reserved = 0;
  }
  if (c.workspace) cudaFree(c.workspace);
  c.workspace = nullptr;
  c.workspace_bytes = 0;
  release_retired_workspaces();
  cudaFree(c.error_flag);
  cudaStreamDestroy(c.stream);
  c = Context();
  return KD_OK;
}

// Reads and clears the device error flag; call after a synchronisation point.
static int check_device_flag() {
  Context& c = ctx();
  int h[4] = {0, 0, 0, 0};
  KD_CUDA_CHECK(cudaMemcpyAsync(h, c.error_flag, sizeof(h), cudaMemcpyDeviceToHost, c.stream));
  KD_CUDA_CHECK(cudaStreamSynchronize(c.stream));
  if (h[0] != 0) {
    cudaMemsetAsync(c.error_flag, 0, sizeof(h), c.stream);
    decode_chain_reset_counters();
    decode_layer_reset_counters();
    return fail(KD_ERR_DEVICE, "a kernel reported error code %d (detail %d, %d, %d)", h[0], h[1], h[2], h[3]);
  }
  return KD_OK;
}

KD_API int kd_synchronize(void) {
  KD_TRY(require_init());
  KD_CUDA_CHECK(cudaStreamSynchronize(ctx().stream));
  return check_device_flag();
}

KD_API int kd_last_error(char* buf, size_t buf_len) {
  if (!buf || buf_len == 0) return KD_ERR_INVALID;
  snprintf(buf, buf_len, "%s", g_last_error.c_str());
  return KD_OK;
}

KD_API int kd_stream(void** stream_out) {
  KD_TRY(require_init());
  if (!stream_out) return fail(KD_ERR_INVALID, "null argument");
  *stream_out = (void*)ctx().stream;
  return KD_OK;
}

KD_API int kd_launch_count(uint64_t* count, int reset) {
  KD_TRY(require_init());
  if (count) *count = ctx().launches;
  if (reset) ctx().launches = 0;
  return KD_OK;
}

KD_API int kd_storage_alloc(uint64_t bytes, int zero, uint64_t* storage_out) {
  KD_TRY(require_init());
  if (!storage_out) return fail(KD_ERR_INVALID, "null argument");
  const uint64_t block = Allocator::round_size(bytes);
  void* p = nullptr;
  uint64_t h;
  {
    std::lock_guard<std::mutex> lk(g_alloc.mu);
    uint64_t actual = 0;  // a reused cached block may be larger than requested
    KD_TRY(g_alloc.alloc_block(block, &p, &actual));
    Storage* s = new Storage{p, bytes, actual, 1};
    h = g_alloc.next_handle++;
    g_alloc.live[h] = s;
  }
  if (zero && bytes) KD_CUDA_CHECK(cudaMemsetAsync(p, 0, bytes, ctx().stream));
  *storage_out = h;
  return KD_OK;
}

KD_API int kd_storage_retain(uint64_t storage) {
  KD_TRY(require_init());
  Storage* s = nullptr;
  KD_TRY(storage_lookup(storage, &s));
  std::lock_guard<std::mutex> lk(g_alloc.mu);
  s->refcount++;
  return KD_OK;
}

KD_API int kd_storage_release(uint64_t storage) {
  KD_TRY(require_init());
  std::lock_guard<std::mutex> lk(g_alloc.mu);
  auto it = g_alloc.live.find(storage);
  if (it == g_alloc.live.end()) return fail(KD_ERR_INVALID, "unknown or released storage handle %llu",
                                            (unsigned long long)storage);
  Storage* s = it->second;
  if (--s->refcount > 0) return KD_OK;
  g_alloc.free_blocks.emplace(s->block_bytes, s->ptr);
  g_alloc.in_use -= s->block_bytes;
  g_alloc.cached += s->block_bytes;
  g_alloc.live.erase(it);
  delete s;
  return KD_OK;
}

KD_API int kd_storage_bytes(uint64_t storage, uint64_t* bytes_out) {
  KD_TRY(require_init());
  Storage* s = nullptr;
  KD_TRY(storage_lookup(storage, &s));
  if (bytes_out) *bytes_out = s->bytes;
  return KD_OK;
}

KD_API int kd_storage_device_ptr(uint64_t storage, void** ptr_out) {
  KD_TRY(require_init());
  Storage* s = nullptr;
  KD_TRY(storage_lookup(storage, &s));
  if (ptr_out) *ptr_out = s->ptr;
  return KD_OK;
}

static int xfer(uint64_t storage, uint64_t off, void* host, uint64_t bytes, bool up, bool sync) {
  KD_TRY(require_init());
  Storage* s = nullptr;
  KD_TRY(storage_lookup(storage, &s));
  KD_REQUIRE(off + bytes <= s->bytes, "transfer of %llu bytes at offset %llu exceeds storage of %llu bytes",
             (unsigned long long)bytes, (unsigned long long)off, (unsigned long long)s->bytes);
  if (bytes == 0) return KD_OK;
  char* d = static_cast<char*>(s->ptr) + off;
  if (up)
    KD_CUDA_CHECK(cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, ctx().stream));
  else
    KD_CUDA_CHECK(cudaMemcpyAsync(host, d, bytes, cudaMemcpyDeviceToHost, ctx().stream));
  if (sync) {
    KD_CUDA_CHECK(cudaStreamSynchronize(ctx().stream));
    if (!up) return check_device_flag();
  }
  return KD_OK;
}

KD_API int kd_upload(uint64_t storage, uint64_t dst_offset_bytes, const void* host, uint64_t bytes) {
  // Pageable host memory: the copy is staged by the runtime before the call returns, so the
  // caller may reuse `host` immediately; synchronise so that behaviour does not depend on it.
  return xfer(storage, dst_offset_bytes, const_cast<void*>(host), bytes, true, true);
}
KD_API int kd_download(uint64_t storage, uint64_t src_offset_bytes, void* host, uint64_t bytes) {
  return xfer(storage, src_offset_bytes, host, bytes, false, true);
}
KD_API int kd_upload_async(uint64_t storage, uint64_t dst_offset_bytes, const void* host, uint64_t bytes) {
  return xfer(storage, dst_offset_bytes, const_cast<void*>(host), bytes, true, false);
}
KD_API int kd_download_async(uint64_t storage, uint64_t src_offset_bytes, void* host, uint64_t bytes) {
  return xfer(storage, src_offset_bytes, host, bytes, false, false);
}

KD_API int kd_host_alloc_pinned(uint64_t bytes, void** host_out) {
  KD_TRY(require_init());
  if (!host_out) return fail(KD_ERR_INVALID, "null argument");
  KD_CUDA_CHECK(cudaHostAlloc(host_out, bytes ? bytes : 1, cudaHostAllocDefault));
  return KD_OK;
}
KD_API int kd_host_free_pinned(void* host) {
  KD_TRY(require_init());
  KD_CUDA_CHECK(cudaFreeHost(host));
  return KD_OK;
}

KD_API int kd_memory_stats(uint64_t* in_use, uint64_t* cached, uint64_t* reserved) {
  KD_TRY(require_init());
  std::lock_guard<std::mutex> lk(g_alloc.mu);
  if (in_use) *in_use = g_alloc.in_use;
  if (cached) *cached = g_alloc.cached;
  if (reserved) *reserved = g_alloc.reserved;
  return KD_OK;
}

KD_API int kd_workspace_bytes(uint64_t* bytes_out) {
  KD_TRY(require_init());
  if (!bytes_out) return fail(KD_ERR_INVALID, "null argument");
  *bytes_out = ctx().workspace_bytes;
  return KD_OK;
}

KD_API int kd_debug_fill_scratch(int byte_value) {
  KD_TRY(require_init());
  Context& c = ctx();
  if (c.workspace) KD_CUDA_CHECK(cudaMemsetAsync(c.workspace, byte_value, c.workspace_bytes, c.stream));
  return attention_decode_static_fill(byte_value);
}

KD_API int kd_empty_cache(void) {
  KD_TRY(require_init());
  KD_CUDA_CHECK(cudaStreamSynchronize(ctx().stream));
  std::lock_guard<std::mutex> lk(g_alloc.mu);
  g_alloc.release_cached();
  return KD_OK;
}

KD_API int kd_event_create(uint64_t* event_out) {
  KD_TRY(require_init());
  if (!event_out) return fail(KD_ERR_INVALID, "null argument");
  cudaEvent_t e;
  KD_CUDA_CHECK(cudaEventCreate(&e));
  *event_out = reinterpret_cast<uint64_t>(e);
  return KD_OK;
}
KD_API int kd_event_record(uint64_t event) {
  KD_TRY(require_init());
  KD_CUDA_CHECK(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), ctx().stream));
  return KD_OK;
}
KD_API int kd_event_elapsed_ms(uint64_t start, uint64_t stop, float* ms_out) {
  KD_TRY(require_init());
  if (!ms_out) return fail(KD_ERR_INVALID, "null argument");
  KD_CUDA_CHECK(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(stop)));
  KD_CUDA_CHECK(cudaEventElapsedTime(ms_out, reinterpret_cast<cudaEvent_t>(start), reinterpret_cast<cudaEvent_t>(stop)));
  return KD_OK;
}
KD_API int kd_event_destroy(uint64_t event) {
  KD_TRY(require_init());
  KD_CUDA_CHECK(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
  return KD_OK;
}

KD_API int kd_set_pdl(int enabled) {
  KD_TRY(require_init());
  ctx().pdl = enabled != 0;
  ctx().pdl_early_kv = enabled == 2;
  return KD_OK;
}
