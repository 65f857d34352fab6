// Device context and the stream-ordered buffer pool.
//
// Reference: pool.rs:36-108 (acquire / release / set_max_pooled_bytes / drain / stats, 256 MiB
// default watermark, power-of-two buckets) and buffer.rs. Differences made for a 180 GB HBM3e
// part: size classes have four steps per octave (a 403 MB score matrix no longer rounds to
// 512 MiB), the default watermark is a fraction of device memory instead of 256 MiB, and the
// backing store is cudaMallocAsync on the runtime's stream, so release -> acquire needs no
// device synchronisation.
#include "runtime.h"
#include "../kernels/kernels.h"
#include <atomic>
#include <cstdlib>
#include <cstring>

namespace ag {

static std::atomic<uint64_t> g_tensor_id{1};
static std::atomic<uint64_t> g_op_id{100000};
static std::atomic<uint64_t> g_fused_id{200000};
uint64_t next_tensor_id() { return g_tensor_id.fetch_add(1, std::memory_order_relaxed); }
uint64_t next_op_id() { return g_op_id.fetch_add(1, std::memory_order_relaxed); }
uint64_t next_fused_id() { return g_fused_id.fetch_add(1, std::memory_order_relaxed); }

DeviceCtx& DeviceCtx::get() {
  static DeviceCtx* ctx = new DeviceCtx();  // never destroyed: outlives every buffer deleter
  return *ctx;
}

static int env_int(const char* name, int dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  return std::atoi(v);
}

static std::atomic<int> g_host_visible_request{-1};   // -1: follow the environment
void DeviceCtx::request_host_visible(bool on) { g_host_visible_request.store(on ? 1 : 0); }

void DeviceCtx::prefetch(const void* ptr, size_t bytes) const {
  if (!host_visible || dry || !ptr || !bytes) return;
  if (cudaMemPrefetchAsync(ptr, bytes, device, stream) != cudaSuccess) cudaGetLastError();   // a hint: the kernels fault pages in otherwise
}

// Backing store of the pool: stream-ordered device memory, or managed memory in host-visible mode.
static cudaError_t backing_alloc(const DeviceCtx& ctx, void** ptr, size_t bytes) {
  if (!ctx.host_visible) return cudaMallocAsync(ptr, bytes, ctx.stream);
  cudaError_t e = cudaMallocManaged(ptr, bytes, cudaMemAttachGlobal);
  if (e == cudaSuccess) ctx.prefetch(*ptr, bytes);
  return e;
}
static void backing_free(const DeviceCtx& ctx, void* ptr) {
  if (!ctx.host_visible) { cudaFreeAsync(ptr, ctx.stream); return; }
  cudaStreamSynchronize(ctx.stream);   // queued kernels may still use the range
  cudaFree(ptr);
}

Status DeviceCtx::init(bool allow_dry) {
  static std::mutex mu;
  std::lock_guard<std::mutex> g(mu);
  if (ready) return Status::OK();
  if (allow_dry && env_int("APPLEGPU_DRY_RUN", 0) == 1) { dry = true; ready = true; name = "dry-run (no device)"; return Status::OK(); }
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    return Status::no_device(std::string("Failed to create CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "no CUDA-capable device"));
  }
  // One process per GPU: APPLEGPU_DEVICE wins, then LOCAL_RANK (torchrun), else device 0.
  int dev = env_int("APPLEGPU_DEVICE", env_int("LOCAL_RANK", 0));
  if (dev < 0 || dev >= count) dev = dev % count;
  e = cudaSetDevice(dev);
  if (e != cudaSuccess) return Status::no_device(std::string("Failed to create CUDA device: ") + cudaGetErrorString(e));
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) return Status::no_device(std::string("Failed to query CUDA device: ") + cudaGetErrorString(e));
  if (prop.major != 10) {
    return Status::no_device(std::string("this library is built for sm_100a only; device is ") + prop.name + " (sm_" +
                             std::to_string(prop.major) + std::to_string(prop.minor) + ")");
  }
  e = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) return Status::no_device(std::string("Failed to create CUDA stream: ") + cudaGetErrorString(e));
  cudaMemPool_t mp;
  if (cudaDeviceGetDefaultMemPool(&mp, dev) == cudaSuccess) {
    uint64_t thr = UINT64_MAX;  // keep freed memory in the pool instead of returning it to the OS
    cudaMemPoolSetAttribute(mp, cudaMemPoolAttrReleaseThreshold, &thr);
  }
  int want_hv = g_host_visible_request.load();
  if (want_hv < 0) want_hv = env_int("APPLEGPU_HOST_VISIBLE", 0);
  if (want_hv == 1) {
    int concurrent = 0;
    cudaDeviceGetAttribute(&concurrent, cudaDevAttrConcurrentManagedAccess, dev);
    if (!concurrent) return Status::no_device("host-visible mode needs concurrent managed access, which this device / driver does not offer");
    host_visible = true;
  }
  device = dev; sm_count = prop.multiProcessorCount; total_mem = prop.totalGlobalMem; name = prop.name;
  // the kernel layer's fixed workspace (status word, skinny-GEMM partials): here, not inside an op call
  Status ws = k::init_device_workspace(stream);
  if (!ws.ok()) return Status::no_device("Failed to create the kernel workspace: " + ws.to_string());
  ready = true;
  return Status::OK();
}

Status DeviceCtx::make_current() const {
  if (dry) return Status::OK();
  int cur = -1;
  if (cudaGetDevice(&cur) == cudaSuccess && cur == device) return Status::OK();
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return Status::compute(std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  return Status::OK();
}

Shared::Shared() : pool(0) {
  DeviceCtx& c = DeviceCtx::get();
  size_t wm;
  int mb = env_int("APPLEGPU_POOL_MB", -1);
  if (mb >= 0) wm = (size_t)mb << 20;
  else wm = c.dry ? ((size_t)256 << 20) : c.total_mem / 4;  // reference default: 256 MiB
  pool.set_max_pooled_bytes(wm);
  int lim = env_int("APPLEGPU_MAX_MEMORY_MB", 0);
  if (lim > 0) pool.set_memory_limit((size_t)lim << 20);
}
Shared& Shared::get() {
  static Shared* s = new Shared();  // never destroyed (see DeviceCtx::get)
  return *s;
}

BufferPool::BufferPool(size_t max_pooled_bytes) : max_pooled_(max_pooled_bytes) {}
BufferPool::~BufferPool() {}

size_t BufferPool::size_class(size_t n) {
  if (n <= 256) return 256;
  if (n <= 4096) { size_t c = 256; while (c < n) c <<= 1; return c; }
  size_t p = 4096;
  while ((p << 1) < n && (p << 1) > p) p <<= 1;  // p < n <= 2p
  if (n <= p) return p;
  size_t step = p / 4;
  return p + ((n - p + step - 1) / step) * step;
}

Status BufferPool::acquire(size_t size, std::shared_ptr<Buffer>* out) {
  DeviceCtx& ctx = DeviceCtx::get();
  size_t cls = size_class(size == 0 ? 4 : size);
  void* ptr = nullptr;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (memory_limit_ && live_bytes_ + cls > memory_limit_) {
      return Status::limit("Memory limit exceeded: " + std::to_string(live_bytes_ + cls) + " bytes requested, limit " + std::to_string(memory_limit_));
    }
    auto it = free_.find(cls);
    if (it != free_.end() && !it->second.empty()) {
      ptr = it->second.back();
      it->second.pop_back();
      if (it->second.empty()) free_.erase(it);
      pooled_bytes_ -= cls;
      hits_++;
    } else {
      misses_++;
      if (fail_next_ > 0) { fail_next_--; return Status::alloc_failed(size); }
    }
  }
  if (ptr) ctx.prefetch(ptr, cls);   // a recycled managed buffer may sit in host memory after a host read
  if (!ptr) {
    if (ctx.dry) {
      std::lock_guard<std::mutex> g(mu_);
      ptr = reinterpret_cast<void*>(fake_ptr_);
      fake_ptr_ += (cls + 255) & ~(size_t)255;
    } else {
      cudaError_t e = backing_alloc(ctx, &ptr, cls);
      if (e != cudaSuccess) {
        cudaGetLastError();
        // Give pooled memory back and retry once before reporting failure.
        drain();
        e = backing_alloc(ctx, &ptr, cls);
        if (e != cudaSuccess) { cudaGetLastError(); return Status::alloc_failed(size); }
      }
    }
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    live_bytes_ += cls; live_buffers_++;
    if (live_bytes_ > peak_live_) peak_live_ = live_bytes_;
  }
  Buffer* b = new Buffer();
  b->ptr = ptr; b->capacity = cls;
  *out = std::shared_ptr<Buffer>(b, [this](Buffer* p) { this->release(p); delete p; });
  return Status::OK();
}

void BufferPool::release(Buffer* b) {
  if (b->borrowed || !b->ptr) return;
  DeviceCtx& ctx = DeviceCtx::get();
  bool keep = false;
  {
    std::lock_guard<std::mutex> g(mu_);
    live_bytes_ -= b->capacity; live_buffers_--;
    if (pooled_bytes_ + b->capacity <= max_pooled_) {
      free_[b->capacity].push_back(b->ptr);
      pooled_bytes_ += b->capacity;
      keep = true;
    }
  }
  if (!keep && !ctx.dry) backing_free(ctx, b->ptr);
}

PoolStats BufferPool::stats() const {
  std::lock_guard<std::mutex> g(mu_);
  PoolStats s;
  s.hits = hits_; s.misses = misses_; s.pooled_bytes = pooled_bytes_; s.bucket_count = free_.size();
  s.live_bytes = live_bytes_; s.peak_live_bytes = peak_live_; s.live_buffers = live_buffers_;
  return s;
}

void BufferPool::drain() {
  DeviceCtx& ctx = DeviceCtx::get();
  std::map<size_t, std::vector<void*>> taken;
  {
    std::lock_guard<std::mutex> g(mu_);
    taken.swap(free_);
    pooled_bytes_ = 0;
  }
  if (ctx.dry) return;
  for (auto& kv : taken) for (void* p : kv.second) backing_free(ctx, p);
}

void BufferPool::set_max_pooled_bytes(size_t n) {
  DeviceCtx& ctx = DeviceCtx::get();
  std::vector<void*> drop;
  {
    std::lock_guard<std::mutex> g(mu_);
    max_pooled_ = n;
    // Evict largest classes first until under the new watermark (pool.rs:77-98).
    while (pooled_bytes_ > max_pooled_ && !free_.empty()) {
      auto it = std::prev(free_.end());
      drop.push_back(it->second.back());
      it->second.pop_back();
      pooled_bytes_ -= it->first;
      if (it->second.empty()) free_.erase(it);
    }
  }
  if (!ctx.dry) for (void* p : drop) backing_free(ctx, p);
}

Status BufferPool::prewarm(const std::vector<size_t>& sizes) {
  std::vector<std::shared_ptr<Buffer>> held;
  for (size_t s : sizes) {
    std::shared_ptr<Buffer> b;
    AG_RETURN_IF_ERROR(acquire(s, &b));
    held.push_back(b);
  }
  return Status::OK();  // buffers return to the free lists as `held` unwinds
}

}  // namespace ag
