// The small all-reduce that ends a product on a row-sharded block, over peer memory.
//
// t(y) %*% X, t(X) %*% X and t(X) %*% (X %*% v) on a matrix whose rows are spread over the GPUs of one node end in a
// sum of nCols (or nCols^2) doubles over the ranks. Through a collective library that costs its launch and
// synchronisation latency (20-35 us measured for 200 doubles with NCCL), a visible share of a 0.7 ms product. Here
// the exchange is one kernel per rank over NVLink peer memory: a rank stores its vector into its slot of every
// peer's buffer, raises a flag there, waits for the flags of all ranks in its own buffer and adds the slots in rank
// order -- every rank forms the same sum in the same order, so all ranks hold identical bits.
//
// Buffers are allocated here (cudaMalloc) and exported with CUDA IPC; the host exchanges the 64-byte handles by its
// own means (the benchmark: torch.distributed all_gather). Plain peer loads and stores only: no multicast objects,
// nothing that outlives a rank in another rank's address space except the mapping itself. Slots are double
// buffered by the parity of the call number, which is enough because a rank cannot be more than one call ahead of
// any peer (it needs every peer's flag of call e before it leaves call e). Every wait is bounded: when a flag does
// not arrive within the time limit the kernel records which rank was missing, fills the result with NaN and returns.
#include "cla_common.cuh"
#include <cstring>
#include <map>

namespace cla {

constexpr int COMM_MAX_WORLD = 16;
constexpr int COMM_THREADS = 1024;

struct CommPeers {
  double* data[COMM_MAX_WORLD];          // peer p's buffer: [2][world][maxDoubles]
  unsigned int* flags[COMM_MAX_WORLD];   // peer p's flags:  [2][world]
};

struct Comm {
  int device = 0, rank = 0, world = 1;
  int64_t maxDoubles = 0;
  char* base = nullptr;       // own allocation: data, then flags, then the error word
  size_t bytes = 0, flagOff = 0, errOff = 0;
  void* opened[COMM_MAX_WORLD] = {};
  CommPeers peers{};
  bool connected = false;
  unsigned int epoch = 0;
  unsigned long long timeoutNs = 2000000000ull;  // 2 s
  std::mutex mu;
};

static std::mutex g_commMu;
static std::map<int64_t, std::shared_ptr<Comm>> g_comms;
static int64_t g_nextComm = 1;

static std::shared_ptr<Comm> comm_lookup(int64_t h) {
  std::lock_guard<std::mutex> lk(g_commMu);
  auto it = g_comms.find(h);
  return it == g_comms.end() ? nullptr : it->second;
}

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One CTA. buf[0..n) in: this rank's partial result; out: the sum over all ranks (rank order).
__global__ void __launch_bounds__(COMM_THREADS, 1)
k_peer_allreduce(CommPeers peers, int rank, int world, int64_t maxDoubles, unsigned int epoch, double* __restrict__ buf,
                 int64_t n, unsigned long long timeoutNs, int* __restrict__ err) {
  const int tid = threadIdx.x;
  const int par = (int)(epoch & 1u);
  __shared__ int missing;
  if (tid == 0) missing = -1;
  // 1. my vector into my slot of every rank's buffer (my own included: the sum then reads one layout)
  for (int p = 0; p < world; p++) {
    double* dst = peers.data[p] + ((size_t)par * world + rank) * maxDoubles;
    for (int64_t i = tid; i < n; i += COMM_THREADS) dst[i] = buf[i];
  }
  __threadfence_system();
  __syncthreads();
  // 2. raise my flag everywhere, then wait for everybody's flag here
  if (tid < world) st_release_sys(peers.flags[tid] + par * world + rank, epoch);
  if (tid < world) {
    const unsigned int* f = peers.flags[rank] + par * world + tid;
    const unsigned long long t0 = now_ns();
    while (ld_acquire_sys(f) != epoch) {
      if (now_ns() - t0 > timeoutNs) {
        atomicMax(&missing, tid);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  if (missing >= 0) {  // a rank never arrived: say which, and make the failure visible in the result
    if (tid == 0) atomicExch(err, 1 + missing);
    for (int64_t i = tid; i < n; i += COMM_THREADS) buf[i] = __longlong_as_double(0x7ff8000000000000ll);
    return;
  }
  // 3. the slots were written by other GPUs: read them past L1
  const double* mine = peers.data[rank] + (size_t)par * world * maxDoubles;
  for (int64_t i = tid; i < n; i += COMM_THREADS) {
    double s = __ldcv(mine + i);
    for (int p = 1; p < world; p++) s += __ldcv(mine + (size_t)p * maxDoubles + i);
    buf[i] = s;
  }
}

static int64_t comm_free(Comm* c) {
  cudaSetDevice(c->device);
  for (int p = 0; p < c->world && p < COMM_MAX_WORLD; p++)
    if (c->opened[p]) cudaIpcCloseMemHandle(c->opened[p]);
  if (c->base) cudaFree(c->base);
  c->base = nullptr;
  return CLA_OK;
}

}  // namespace cla

using namespace cla;

extern "C" {

int64_t cla_comm_create(int32_t device, int32_t rank, int32_t world, int64_t maxDoubles, void* ipcHandleOut) {
  if (world < 1 || world > COMM_MAX_WORLD || rank < 0 || rank >= world || maxDoubles < 1 || maxDoubles > (1 << 24))
    return fail(CLA_ERR_BAD_ARG, "comm_create: world in [1, 16], rank in [0, world), maxDoubles in [1, 2^24]");
  if (!ipcHandleOut) return fail(CLA_ERR_BAD_ARG, "comm_create: null handle buffer");
  static_assert(sizeof(cudaIpcMemHandle_t) == CLA_COMM_HANDLE_BYTES, "IPC handle size");
  CLA_CUDA(cudaSetDevice(device));
  auto c = std::make_shared<Comm>();
  c->device = device;
  c->rank = rank;
  c->world = world;
  c->maxDoubles = maxDoubles;
  const size_t dataBytes = (size_t)2 * world * maxDoubles * sizeof(double);
  c->flagOff = (dataBytes + 255) & ~(size_t)255;
  c->errOff = c->flagOff + 256;
  c->bytes = c->errOff + 256;
  CLA_CUDA(cudaMalloc((void**)&c->base, c->bytes));
  CLA_CUDA(cudaMemset(c->base, 0, c->bytes));
  CLA_CUDA(cudaDeviceSynchronize());
  cudaIpcMemHandle_t hdl;
  cudaError_t e = cudaIpcGetMemHandle(&hdl, c->base);
  if (e != cudaSuccess) {
    comm_free(c.get());
    return fail(CLA_ERR_CUDA, std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
  }
  memcpy(ipcHandleOut, &hdl, sizeof(hdl));
  std::lock_guard<std::mutex> lk(g_commMu);
  const int64_t h = g_nextComm++;
  g_comms[h] = c;
  return h;
}

int64_t cla_comm_connect(int64_t comm, const void* allHandles) {
  auto c = comm_lookup(comm);
  if (!c) return fail(CLA_ERR_BAD_HANDLE, "unknown comm handle");
  std::lock_guard<std::mutex> lk(c->mu);
  if (c->connected) return fail(CLA_ERR_STATE, "comm_connect: already connected");
  CLA_CUDA(cudaSetDevice(c->device));
  for (int p = 0; p < c->world; p++) {
    char* b = c->base;
    if (allHandles && p != c->rank) {  // null: every rank maps to this rank's own buffer (single-process checks)
      cudaIpcMemHandle_t hdl;
      memcpy(&hdl, (const char*)allHandles + (size_t)p * sizeof(hdl), sizeof(hdl));
      void* ptr = nullptr;
      cudaError_t e = cudaIpcOpenMemHandle(&ptr, hdl, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) return fail(CLA_ERR_CUDA, std::string("cudaIpcOpenMemHandle (rank ") + std::to_string(p) + "): " + cudaGetErrorString(e));
      c->opened[p] = ptr;
      b = (char*)ptr;
    }
    c->peers.data[p] = (double*)b;
    c->peers.flags[p] = (unsigned int*)(b + c->flagOff);
  }
  c->connected = true;
  return CLA_OK;
}

int64_t cla_comm_set_timeout_ms(int64_t comm, int64_t ms) {
  auto c = comm_lookup(comm);
  if (!c) return fail(CLA_ERR_BAD_HANDLE, "unknown comm handle");
  if (ms < 1 || ms > 60000) return fail(CLA_ERR_BAD_ARG, "comm_set_timeout_ms: 1..60000");
  std::lock_guard<std::mutex> lk(c->mu);
  c->timeoutNs = (unsigned long long)ms * 1000000ull;
  return CLA_OK;
}

int64_t cla_allreduce_dev(int64_t comm, double* dBuf, int64_t n, void* stream) {
  auto c = comm_lookup(comm);
  if (!c) return fail(CLA_ERR_BAD_HANDLE, "unknown comm handle");
  std::lock_guard<std::mutex> lk(c->mu);
  if (!c->connected) return fail(CLA_ERR_STATE, "allreduce: cla_comm_connect has not been called");
  if (n < 0 || n > c->maxDoubles) return fail(CLA_ERR_SHAPE, "allreduce: more doubles than the comm was created for");
  if (!dBuf && n) return fail(CLA_ERR_BAD_ARG, "allreduce: null buffer");
  CLA_CUDA(cudaSetDevice(c->device));
  c->epoch++;
  if (c->epoch == 0) c->epoch = 2;  // flags start at 0: never wait for 0; keeps the parity sequence
  k_peer_allreduce<<<1, COMM_THREADS, 0, (cudaStream_t)stream>>>(c->peers, c->rank, c->world, c->maxDoubles, c->epoch, dBuf, n,
                                                              c->timeoutNs, (int*)(c->base + c->errOff));
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

int64_t cla_comm_status(int64_t comm) {
  auto c = comm_lookup(comm);
  if (!c) return fail(CLA_ERR_BAD_HANDLE, "unknown comm handle");
  std::lock_guard<std::mutex> lk(c->mu);
  CLA_CUDA(cudaSetDevice(c->device));
  int e = 0;
  CLA_CUDA(cudaDeviceSynchronize());  // the kernels may sit on non-blocking streams
  CLA_CUDA(cudaMemcpy(&e, c->base + c->errOff, sizeof(e), cudaMemcpyDeviceToHost));
  if (e != 0) {
    CLA_CUDA(cudaMemset(c->base + c->errOff, 0, sizeof(e)));
    return fail(CLA_ERR_DEVICE_CHECK, "allreduce: rank " + std::to_string(e - 1) + " did not arrive within the time limit");
  }
  return CLA_OK;
}

int64_t cla_comm_destroy(int64_t comm) {
  std::shared_ptr<Comm> c;
  {
    std::lock_guard<std::mutex> lk(g_commMu);
    auto it = g_comms.find(comm);
    if (it == g_comms.end()) return fail(CLA_ERR_BAD_HANDLE, "unknown comm handle");
    c = it->second;
    g_comms.erase(it);
  }
  std::lock_guard<std::mutex> lk(c->mu);
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  return comm_free(c.get());
}

}  // extern "C"
