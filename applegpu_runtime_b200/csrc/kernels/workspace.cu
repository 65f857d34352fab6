// Fixed per-process device workspace of the kernel layer, created once when the device context is
// set up (never lazily inside an op call, which would be a synchronising allocation in the middle of
// a stream-ordered forward):
//   * the pipeline status word of the tcgen05 kernels (a bounded wait that gives up records a code
//     there) with a pinned host mirror, so a synchronisation point can read it with a plain load;
//   * the partial-sum workspace and the slab counters of the skinny GEMM;
//   * the arrival counters and the tile lists of the chained tensor-core products.
// Also holds the test-only kernel that lets a bounded wait run out on purpose: it waits on an mbarrier
// that nothing arrives at, with a limit of about a millisecond, records its code and returns.
#include "common.cuh"
#include "sm100.cuh"
#include <mutex>

namespace ag { namespace k {

namespace {
constexpr int kStatusSlots = 128;            // pinned mirror: slot 0 for blocking checks, the rest for markers
constexpr size_t kStatusRegion = 256;        // the status word sits alone in its 256-byte line
constexpr size_t kSkCounterBytes = (65536 / 64) * sizeof(unsigned int);
constexpr size_t kSkPartialBytes = ((size_t)1 << 18) * 16 * sizeof(float);   // k_slabs * n * 16 rows of fp32
constexpr size_t kChainFlagBytes = ((size_t)kChainMax * kChainFlagStride + 64) * sizeof(int);   // counters + the exit counter
constexpr size_t kChainArenaBytes = (size_t)kChainArenaInts * sizeof(int);

uint8_t* g_block = nullptr;
int* g_status_host = nullptr;
std::mutex g_mu;
}  // namespace

Status init_device_workspace(cudaStream_t s) {
  std::lock_guard<std::mutex> g(g_mu);
  if (g_block) return Status::OK();
  // status word | skinny counters | chain counters (these three are cleared) | skinny partials | chain tile lists
  const size_t total = kStatusRegion + kSkCounterBytes + kChainFlagBytes + kSkPartialBytes + kChainArenaBytes;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, total);
  if (e != cudaSuccess) return cuda_status(e, "kernel workspace");
  e = cudaMemsetAsync(p, 0, kStatusRegion + kSkCounterBytes + kChainFlagBytes, s);
  if (e != cudaSuccess) { cudaFree(p); return cuda_status(e, "kernel workspace clear"); }
  void* h = nullptr;
  e = cudaMallocHost(&h, kStatusSlots * sizeof(int));
  if (e != cudaSuccess) { cudaFree(p); return cuda_status(e, "pinned status mirror"); }
  g_status_host = static_cast<int*>(h);
  for (int i = 0; i < kStatusSlots; i++) g_status_host[i] = 0;
  g_block = static_cast<uint8_t*>(p);
  return Status::OK();
}

int* matmul_status_word() { return reinterpret_cast<int*>(g_block); }
unsigned int* skinny_counters() { return g_block ? reinterpret_cast<unsigned int*>(g_block + kStatusRegion) : nullptr; }
int* chain_flags() { return g_block ? reinterpret_cast<int*>(g_block + kStatusRegion + kSkCounterBytes) : nullptr; }
float* skinny_partials() { return g_block ? reinterpret_cast<float*>(g_block + kStatusRegion + kSkCounterBytes + kChainFlagBytes) : nullptr; }
int* chain_arena() { return g_block ? reinterpret_cast<int*>(g_block + kStatusRegion + kSkCounterBytes + kChainFlagBytes + kSkPartialBytes) : nullptr; }
int status_slots() { return kStatusSlots; }

// Enqueues a copy of the status word into pinned slot `slot`; the value is defined once the stream
// (or an event recorded after this call) has been waited for.
Status status_snapshot(cudaStream_t s, int slot) {
  if (!g_block || !g_status_host || slot < 0 || slot >= kStatusSlots) return Status::OK();
  cudaError_t e = cudaMemcpyAsync(g_status_host + slot, g_block, sizeof(int), cudaMemcpyDeviceToHost, s);
  return cuda_status(e, "status snapshot");
}
// Reads a snapshot the caller has waited for. A non-zero value also clears the device word (stream-
// ordered), so that the kernels that follow start from a clean state.
int status_take(cudaStream_t s, int slot) {
  if (!g_block || !g_status_host || slot < 0 || slot >= kStatusSlots) return 0;
  int v = g_status_host[slot];
  if (v != 0) {
    g_status_host[slot] = 0;
    cudaMemsetAsync(g_block, 0, sizeof(int), s);
  }
  return v;
}

// Reads and clears the pipeline status word; non-zero means a bounded wait gave up. Waits for the stream.
int matmul_take_status(cudaStream_t s) {
  if (!g_block) return 0;
  if (!status_snapshot(s, 0).ok()) return -1;
  if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
  return status_take(s, 0);
}

// ── a wait that runs out, for tests ─────────────────────────────────────────
// One thread waits on a freshly initialised mbarrier whose phase nobody completes. The limit is
// `limit_ns` (about a millisecond in the test), after which the wait records `code` in the status
// word and the kernel returns: the same path a mis-programmed pipeline takes, without a fault, a
// trap or an unbounded loop.
__global__ void wait_runs_out_kernel(int* status, int code, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 1);
    sm100::mbar_fence_init();
    const unsigned long long t0 = sm100::globaltimer_ns();
    uint32_t spins = 0;
    while (!sm100::mbar_try_wait(&bar, 0)) {
      if ((++spins & 0xff) == 0 && sm100::globaltimer_ns() - t0 > limit_ns) { atomicCAS(status, 0, code); break; }
      if (spins > (1u << 26)) { atomicCAS(status, 0, code); break; }   // second bound, in iterations
    }
  }
}
Status launch_wait_runs_out(cudaStream_t s, int code, unsigned long long limit_ns) {
  if (!g_block) return Status::compute("kernel workspace is not initialised");
  if (limit_ns > 50000000ull) limit_ns = 50000000ull;   // never more than 50 ms
  wait_runs_out_kernel<<<1, 32, 0, s>>>(matmul_status_word(), code, limit_ns);
  AG_CHECK_LAUNCH("wait_runs_out");
  return Status::OK();
}

}}  // namespace ag::k
