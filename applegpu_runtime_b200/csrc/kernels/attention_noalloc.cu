// Attention for callers that must not allocate device memory.
//
// The regular attention path (exec.cc, attention_exec) takes its [batch*heads, q_len, kv_len]
// score matrix from the buffer pool, which may call cudaMallocAsync. Some hosts of this library
// cannot do that at the point where they need attention: code running inside a region where the
// CUDA allocator is off limits (a real-time serving loop with a fixed memory budget, a plugin
// that was handed its buffers by the embedding application and is forbidden to grow the
// process's device footprint, a library called between another framework's allocator
// checkpoints). For them this file provides one entry point that takes only caller-owned
// input/output pointers and keeps its scratch in a fixed array that is part of the library image.
//
// The array lives in device memory of every GPU that loads the library, from load until exit.
// In host code its name is only a handle: the device address comes from cudaGetSymbolAddress,
// asked once per device with that device current, and that pointer is what the kernels receive.
#include "common.cuh"
#include <mutex>
#include "../../../include/applegpu_b200_ext.h"

namespace ag {
void set_ffi_error_text(const std::string& m);  // ffi.cc: feeds applegpu_ffi_last_error()
namespace k {
Status matmul_with_status(cudaStream_t s, const GemmDesc& d, int* status_word);
}
}

namespace {

constexpr size_t kScratchBytes = APPLEGPU_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];
static __device__ __align__(256) int g_noalloc_status[64];

constexpr int kMaxDevices = 64;
struct DeviceSlots { void* scratch = nullptr; int* status = nullptr; bool ready = false; };
DeviceSlots g_slots[kMaxDevices];
std::mutex g_slots_mu;

// First call on a device resolves the two symbols; later calls reuse the pointers.
// The device the first successful call saw (-1 before that).
int g_first_device = -1;
int first_device_seen() { std::lock_guard<std::mutex> g(g_slots_mu); return g_first_device; }

ag::Status slots_for_current_device(DeviceSlots** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return ag::Status::compute(std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return ag::Status::compute("device ordinal out of range");
  std::lock_guard<std::mutex> g(g_slots_mu);
  DeviceSlots& sl = g_slots[dev];
  if (!sl.ready) {
    void* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return ag::Status::compute(std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
    void* st = nullptr;
    e = cudaGetSymbolAddress((void**)&st, g_noalloc_status);
    if (e != cudaSuccess) return ag::Status::compute(std::string("cudaGetSymbolAddress(status): ") + cudaGetErrorString(e));
    sl.scratch = p; sl.status = reinterpret_cast<int*>(st); sl.ready = true;
    if (g_first_device < 0) g_first_device = dev;
  }
  *out = &sl;
  return ag::Status::OK();
}

}  // namespace

extern "C" int32_t applegpu_attention_noalloc(const void* q, const void* k, const void* v, void* out, int8_t dtype,
                                              uint64_t batch_heads, uint64_t q_len, uint64_t kv_len, uint64_t d_k, uint64_t d_v,
                                              bool causal, void* cuda_stream) {
  using namespace ag;
  auto fail = [](const std::string& m) { set_ffi_error_text("attention_noalloc failed: " + m); return -1; };
  DType dt;
  if (!dtype_from_wire(dtype, &dt) || !(dt == DType::F32 || dt == DType::F16 || dt == DType::BF16))
    return fail("dtype must be float32, float16 or bfloat16");
  if (!q || !k || !v || !out) return fail("null tensor pointer");
  if (batch_heads == 0 || q_len == 0 || d_v == 0) return 0;  // empty output
  if (kv_len == 0 || d_k == 0) return fail("kv_len and d_k must be non-zero");
  const size_t esz = dtype_size(dt);
  // scores: [batch_heads, q_len, kv_len] in the storage dtype
  const long double need = (long double)batch_heads * (long double)q_len * (long double)kv_len * (long double)esz;
  if (need > (long double)kScratchBytes)
    return fail("score matrix of " + std::to_string((unsigned long long)need) + " bytes exceeds the built-in scratch of " +
                std::to_string((unsigned long long)kScratchBytes) + " bytes (batch_heads * q_len * kv_len * element size)");
  DeviceSlots* sl = nullptr;
  Status s = slots_for_current_device(&sl);
  if (!s.ok()) return fail(s.to_string());
  {
    // The kernels' one-time setup (shared-memory opt-in, SM count) is held per process, for the device
    // the process first used: a call with another device current is refused instead of mis-launched.
    int cur = -1, first = first_device_seen();
    cudaGetDevice(&cur);
    if (first >= 0 && cur != first)
      return fail("this process already runs kernels on device " + std::to_string(first) + "; one process serves one GPU (current device is " + std::to_string(cur) + ")");
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);

  // The scratch keeps whatever the previous call left; every score element is rewritten by the
  // first GEMM before it is read, and the pipeline status word is the only thing that must start at zero.
  cudaError_t e = cudaMemsetAsync(sl->status, 0, sizeof(int), stream);
  if (e != cudaSuccess) return fail(std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));

  const int64_t bh = (int64_t)batch_heads, tq = (int64_t)q_len, tk = (int64_t)kv_len, dk = (int64_t)d_k, dv = (int64_t)d_v;
  k::GemmDesc g1;
  g1.dtype = dt; g1.b_dtype = dt;
  g1.a = q; g1.b = k; g1.c = sl->scratch;
  g1.m = tq; g1.n = tk; g1.k = dk; g1.batch = bh; g1.batch_inner = 1;
  g1.a_row = dk; g1.a_col = 1; g1.a_batch = tq * dk;
  g1.b_row = 1; g1.b_col = dk; g1.b_batch = tk * dk;          // K^T read in place (K-major operand)
  g1.c_row = tk; g1.c_batch = tq * tk;
  g1.ep.alpha = 1.0f / sqrtf((float)dk);
  s = k::matmul_with_status(stream, g1, sl->status);
  if (!s.ok()) return fail(s.to_string());
  TView scores = TView::make(sl->scratch, dt, {bh, tq, tk});
  s = k::softmax(stream, scores, causal, scores);
  if (!s.ok()) return fail(s.to_string());
  k::GemmDesc g2;
  g2.dtype = dt; g2.b_dtype = dt;
  g2.a = sl->scratch; g2.b = v; g2.c = out;
  g2.m = tq; g2.n = dv; g2.k = tk; g2.batch = bh; g2.batch_inner = 1;
  g2.a_row = tk; g2.a_col = 1; g2.a_batch = tq * tk;
  g2.b_row = dv; g2.b_col = 1; g2.b_batch = tk * dv;
  g2.c_row = dv; g2.c_batch = tq * dv;
  s = k::matmul_with_status(stream, g2, sl->status);
  if (!s.ok()) return fail(s.to_string());
  return 0;
}

// The tensor-core GEMMs inside applegpu_attention_noalloc bound every wait; one that gives up leaves a
// code in this entry point's own status word (not the one applegpu_pipeline_status reads) and `out`
// undefined. This reads that word back without allocating: it waits for `cuda_stream`, then copies the
// four bytes into a local variable. 0 = the last call on this device ran to completion; a positive
// value = the code of the wait that timed out; -1 = the query itself failed (see last_error).
extern "C" int32_t applegpu_attention_noalloc_status(void* cuda_stream) {
  using namespace ag;
  auto fail = [](const std::string& m) { set_ffi_error_text("attention_noalloc_status failed: " + m); return -1; };
  DeviceSlots* sl = nullptr;
  Status s = slots_for_current_device(&sl);
  if (!s.ok()) return fail(s.to_string());
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  cudaError_t e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(std::string("cudaStreamSynchronize: ") + cudaGetErrorString(e));
  int v = 0;
  e = cudaMemcpy(&v, sl->status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(std::string("cudaMemcpy: ") + cudaGetErrorString(e));
  return v;
}
