// Handle life cycle: group registration, upload, skip-index construction, and the device decode
// kernels that turn the reference's index structures into row ids (used by the bit-exact checks
// and, for RLE / OLE, once at upload to build the row-ordered forms the product kernels read).
#include "cla_common.cuh"
#include <cmath>
#include <cub/cub.cuh>
#include <algorithm>
#include <cstring>
#include <map>
#include <memory>

namespace cla {

static thread_local std::string g_lastError;
void set_error(const std::string& msg) { g_lastError = msg; }
int64_t fail(int64_t code, const std::string& msg) {
  g_lastError = msg;
  return code;
}
const std::string& last_error() { return g_lastError; }

static std::mutex g_tabMu;
static std::map<int64_t, std::shared_ptr<Matrix>> g_table;
static int64_t g_next = 1;

std::shared_ptr<Matrix> lookup(cla_handle h) {
  std::lock_guard<std::mutex> lk(g_tabMu);
  auto it = g_table.find(h);
  return it == g_table.end() ? nullptr : it->second;
}

static int64_t grow(void** p, size_t* cur, size_t bytes) {
  if (bytes <= *cur) return CLA_OK;
  if (*p) cudaFree(*p);
  *p = nullptr;
  *cur = 0;
  size_t want = bytes + bytes / 4 + 256;
  cudaError_t e = cudaMalloc(p, want);
  if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc scratch: ") + cudaGetErrorString(e));
  *cur = want;
  return CLA_OK;
}
int64_t order_begin(Matrix* m, cudaStream_t s) {
  if (m->lastValid && m->lastStream != s) CLA_CUDA(cudaStreamWaitEvent(s, m->lastDone, 0));
  return CLA_OK;
}
int64_t order_end(Matrix* m, cudaStream_t s) {
  CLA_CUDA(cudaEventRecord(m->lastDone, s));
  m->lastStream = s;
  m->lastValid = true;
  return CLA_OK;
}
int64_t ensure_scratch(Matrix* m, size_t bytes) { return grow(&m->scratch, &m->scratchBytes, bytes); }
int64_t ensure_scratch2(Matrix* m, size_t bytes) { return grow(&m->scratch2, &m->scratch2Bytes, bytes); }
int64_t ensure_io(Matrix* m, size_t bytes) { return grow(&m->io, &m->ioBytes, bytes); }
int64_t ensure_small(Matrix* m, size_t bytes) { return grow(&m->small_, &m->smallBytes, bytes); }

constexpr size_t PROF_MAX = 512;
void prof_begin(Matrix* m, cudaStream_t s) {
  if (!m->profile || m->profUsed >= PROF_MAX) return;
  if (m->profUsed == m->profEvents.size()) {
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
    m->profEvents.push_back({a, b});
  }
  cudaEventRecord(m->profEvents[m->profUsed].first, s);
}
void prof_end(Matrix* m, cudaStream_t s) {
  if (!m->profile || m->profUsed >= m->profEvents.size()) return;
  cudaEventRecord(m->profEvents[m->profUsed].second, s);
  m->profUsed++;
}
void prof_collect(Matrix* m) {
  for (size_t i = 0; i < m->profUsed; i++) {
    float ms = 0;
    if (cudaEventSynchronize(m->profEvents[i].second) == cudaSuccess &&
        cudaEventElapsedTime(&ms, m->profEvents[i].first, m->profEvents[i].second) == cudaSuccess) {
      m->stats.main_kernel_ms += ms;
      m->stats.main_kernel_count++;
    }
  }
  m->profUsed = 0;
}

// ------------------------------------------------------------------------------------------------
// device kernels used at upload and for decode checks
// ------------------------------------------------------------------------------------------------

// One warp per value k: prefix-sum the (gap, len) pairs into absolute runs
// (decode rule of ColGroupRLE.java:114-117: start = prevEnd + gap, end = start + len).
__global__ void k_rle_decode(const int32_t* __restrict__ ptr, const uint16_t* __restrict__ data, int nVals,
                             RleRun* __restrict__ runs, uint32_t* __restrict__ keys, int nRows, int32_t* err) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= nVals) return;
  const int p0 = ptr[warp] >> 1, p1 = ptr[warp + 1] >> 1;
  int base = 0;
  for (int p = p0; p < p1; p += 32) {
    const int i = p + lane;
    int gap = 0, len = 0;
    if (i < p1) {
      gap = data[2 * i];
      len = data[2 * i + 1];
    }
    int s = gap + len;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += t;
    }
    const int end = base + s;
    if (i < p1) {
      RleRun r;
      r.start = end - len;
      r.len = (uint16_t)len;
      r.k = (uint16_t)warp;
      runs[i] = r;
      keys[i] = len > 0 ? (uint32_t)r.start : 0xFFFFFFFFu;
      if (end > nRows) atomicExch(err, 1);  // run past the end of the matrix
    }
    base = __shfl_sync(0xffffffffu, end, 31);
  }
}

__global__ void k_rle_gather(const RleRun* __restrict__ in, const uint32_t* __restrict__ idx, RleRun* __restrict__ out,
                             int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) out[i] = in[idx[i]];
}

__global__ void k_iota(uint32_t* p, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) p[i] = (uint32_t)i;
}

// runSkip[b] = first run (row order) whose end lies behind row b * SKIP_ROWS
__global__ void k_rle_skip(const RleRun* __restrict__ runs, int64_t nRuns, int32_t* __restrict__ skip, int nBlocks) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nBlocks) return;
  const int row = b * SKIP_ROWS;
  int64_t lo = 0, hi = nRuns;
  while (lo < hi) {
    int64_t mid = (lo + hi) >> 1;
    if (runs[mid].start + (int)runs[mid].len > row) hi = mid;
    else lo = mid + 1;
  }
  skip[b] = (int32_t)lo;
}

// One warp per value k walks its OLE segments ([n, o_1..o_n] per 65535-row window,
// ColGroupOLE.java:558-599) and writes k into the per-row map.
template <typename T>
__global__ void k_ole_to_map(const int32_t* __restrict__ ptr, const uint16_t* __restrict__ data, int nVals,
                             T* __restrict__ map, int nRows, int32_t* err) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= nVals) return;
  const int boff = ptr[warp], blen = ptr[warp + 1] - ptr[warp];
  int seg = 0;
  for (int bix = 0; bix < blen; seg++) {
    const int n = data[boff + bix];
    const int64_t base = (int64_t)seg * BITMAP_BLOCK_SZ;
    for (int j = lane; j < n; j += 32) {
      const int64_t r = base + data[boff + bix + 1 + j];
      if (r < nRows) map[r] = (T)warp;
      else atomicExch(err, 2);
    }
    bix += n + 1;
  }
}

template <typename T>
__global__ void k_fill(T* p, T v, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) p[i] = v;
}

// ids of a dense map (DDC, or transcoded OLE with `sentinel` meaning "no tuple")
__global__ void k_decode_map(DevGroup g, int sentinel, int32_t* __restrict__ ids, int nRows) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < nRows; i += stride) {
    int id = map_get(g.mapType, g.map, g.mapHi, i);
    ids[i] = (id == sentinel) ? -1 : id;
  }
}

__global__ void k_decode_sdc(DevGroup g, int32_t* __restrict__ ids, int nRows) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nBlocks = (nRows + SKIP_ROWS - 1) / SKIP_ROWS;
  if (warp >= nBlocks) return;
  const int rb = warp * SKIP_ROWS, re = min(nRows, rb + SKIP_ROWS);
  sdc_walk_block(g, rb, re, [&](int row, int e) { ids[row] = g.single ? 0 : map_get(g.mapType, g.map, g.mapHi, e); });
}

__global__ void k_decode_runs(const RleRun* __restrict__ runs, int64_t nRuns, int32_t* __restrict__ ids) {
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= nRuns) return;
  const RleRun r = runs[warp];
  for (int i = lane; i < r.len; i += 32) ids[r.start + i] = r.k;
}

__global__ void k_iota_i32(int32_t* p, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = i;
}

// counts ------------------------------------------------------------------------------------------
__global__ void k_counts_map(DevGroup g, int sentinel, unsigned long long* __restrict__ counts) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < g.mapSize; i += stride) {
    int id = map_get(g.mapType, g.map, g.mapHi, i);
    if (id != sentinel) atomicAdd(&counts[id], 1ULL);
  }
}
// RLE: counts[k] = sum of run lengths (ColGroupRLE.java:259-265), from the registered arrays
__global__ void k_counts_rle(const int32_t* __restrict__ ptr, const uint16_t* __restrict__ data, int nVals,
                             unsigned long long* __restrict__ counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= nVals) return;
  unsigned long long s = 0;
  for (int p = (ptr[warp] >> 1) + lane; p < (ptr[warp + 1] >> 1); p += 32) s += data[2 * p + 1];
  for (int d = 16; d; d >>= 1) s += __shfl_down_sync(0xffffffffu, s, d);
  if (lane == 0) counts[warp] = s;
}
// OLE: counts[k] = sum of the segment headers (ColGroupOLE.java:152-169)
__global__ void k_counts_ole(const int32_t* __restrict__ ptr, const uint16_t* __restrict__ data, int nVals,
                             unsigned long long* __restrict__ counts) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= nVals) return;
  const int boff = ptr[k], blen = ptr[k + 1] - ptr[k];
  unsigned long long s = 0;
  for (int bix = 0; bix < blen; bix += data[boff + bix] + 1) s += data[boff + bix];
  counts[k] = s;
}

__global__ void k_count_nnz(const double* __restrict__ d, int64_t n, unsigned long long* __restrict__ out) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  unsigned long long c = 0;
  for (; i < n; i += stride) c += (d[i] != 0.0);
  for (int s = 16; s; s >>= 1) c += __shfl_down_sync(0xffffffffu, c, s);
  if ((threadIdx.x & 31) == 0 && c) atomicAdd(out, c);
}

__global__ void k_scale_rows(double* __restrict__ u, const double* __restrict__ w, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) u[i] *= w[i];
}

static inline int grid_for(int64_t n, int block, int cap = 148 * 16) {
  int64_t g = (n + block - 1) / block;
  return (int)std::max<int64_t>(1, std::min<int64_t>(g, cap));
}

int64_t launch_count_nnz(Matrix* m, const double* d, int64_t n, unsigned long long* dCount, cudaStream_t s) {
  CLA_CUDA(cudaMemsetAsync(dCount, 0, sizeof(unsigned long long), s));
  if (n > 0) k_count_nnz<<<grid_for(n, 256), 256, 0, s>>>(d, n, dCount);
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

int64_t launch_scale_rows(Matrix* m, double* dU, const double* dW, int64_t n, cudaStream_t s) {
  if (n > 0) k_scale_rows<<<grid_for(n, 256), 256, 0, s>>>(dU, dW, n);
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

static int sentinel_of(const DevGroup& g) { return g.origType == GT_OLE ? g.nVals - 1 : -1; }

int64_t launch_group_decode(Matrix* m, int gi, int32_t* dIds, cudaStream_t s) {
  const DevGroup& g = m->groups[gi];
  const int n = m->nRows;
  if (n == 0) return CLA_OK;
  switch (g.type) {
    case GT_DDC: k_decode_map<<<grid_for(n, 256), 256, 0, s>>>(g, sentinel_of(g), dIds, n); break;
    case GT_SDC: {
      k_fill<int32_t><<<grid_for(n, 256), 256, 0, s>>>(dIds, -1, n);
      const int nb = (n + SKIP_ROWS - 1) / SKIP_ROWS;
      k_decode_sdc<<<(nb * 32 + 255) / 256, 256, 0, s>>>(g, dIds, n);
      break;
    }
    case GT_RLE:
      k_fill<int32_t><<<grid_for(n, 256), 256, 0, s>>>(dIds, -1, n);
      if (g.nRuns) k_decode_runs<<<(unsigned)((g.nRuns * 32 + 255) / 256), 256, 0, s>>>(g.runs, g.nRuns, dIds);
      break;
    case GT_UNC: k_iota_i32<<<(n + 255) / 256, 256, 0, s>>>(dIds, n); break;
    default: return fail(CLA_ERR_UNSUPPORTED, "decode: unsupported group type");
  }
  m->stats.kernel_launches += 2;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

int64_t launch_group_counts(Matrix* m, int gi, unsigned long long* dCounts, cudaStream_t s) {
  const DevGroup& g = m->groups[gi];
  const int nv = g.origType == GT_OLE ? g.nVals - 1 : g.nVals;
  CLA_CUDA(cudaMemsetAsync(dCounts, 0, sizeof(unsigned long long) * std::max(nv, 1), s));
  if (g.origType == GT_OLE) {
    if (nv) k_counts_ole<<<(nv + 127) / 128, 128, 0, s>>>(g.ptr, g.data, nv, dCounts);
  } else if (g.type == GT_RLE) {
    if (nv) k_counts_rle<<<(nv * 32 + 255) / 256, 256, 0, s>>>(g.ptr, g.data, nv, dCounts);
  } else if (g.type == GT_DDC || (g.type == GT_SDC && !g.single)) {
    if (g.mapSize) k_counts_map<<<grid_for(g.mapSize, 256), 256, 0, s>>>(g, -1, dCounts);
  } else if (g.type == GT_SDC) {
    unsigned long long c = (unsigned long long)g.nOff;
    CLA_CUDA(cudaMemcpyAsync(dCounts, &c, sizeof(c), cudaMemcpyHostToDevice, s));
    CLA_CUDA(cudaStreamSynchronize(s));
  } else
    return fail(CLA_ERR_UNSUPPORTED, "counts: group has no dictionary");
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

// ids of a map registered from device memory must stay below nVals (host-registered maps are checked on the host)
__global__ void k_check_ids(int mapType, const void* __restrict__ map, int64_t n, int nVals, int32_t* err) {
  bool bad = false;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    bad |= map_get(mapType, map, nullptr, i) >= nVals;
  if (bad) atomicExch(err, 3);
}

// ------------------------------------------------------------------------------------------------
// upload
// ------------------------------------------------------------------------------------------------
template <typename T>
static int64_t upload(Matrix* m, const T* src, size_t n, const T** dst, bool index) {
  *dst = nullptr;
  if (n == 0) return CLA_OK;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, n * sizeof(T));
  if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc: ") + cudaGetErrorString(e));
  m->allocs.push_back(p);
  m->deviceBytes += n * sizeof(T);
  if (index) m->indexBytes += n * sizeof(T);
  CLA_CUDA(cudaMemcpy(p, src, n * sizeof(T), cudaMemcpyHostToDevice));
  *dst = (const T*)p;
  return CLA_OK;
}

template <typename T>
static int64_t dev_alloc(Matrix* m, size_t n, T** dst) {
  *dst = nullptr;
  if (n == 0) return CLA_OK;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, n * sizeof(T));
  if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc: ") + cudaGetErrorString(e));
  m->allocs.push_back(p);
  m->deviceBytes += n * sizeof(T);
  *dst = (T*)p;
  return CLA_OK;
}

static size_t map_bytes(int mapType, int64_t size, size_t* hiBytes) {
  *hiBytes = 0;
  switch (mapType) {
    case CLA_MAP_ZERO: return 0;
    case CLA_MAP_BIT: return (size_t)((size + 63) / 64) * 8;
    case CLA_MAP_UBYTE:
    case CLA_MAP_BYTE: return (size_t)size;
    case CLA_MAP_CHAR: return (size_t)size * 2;
    case CLA_MAP_CHAR_BYTE: *hiBytes = (size_t)size; return (size_t)size * 2;
    case CLA_MAP_INT: return (size_t)size * 4;
    default: return 0;
  }
}

// Host pass over an offset stream that records, for every SKIP_ROWS boundary, where decoding can
// resume (the role of AOffset's skip list, AOffset.java:79,177-199). Also validates the stream.
static int64_t build_sdc_skip(const HostGroup& hg, int nRows, std::vector<SdcSkip>& skip) {
  const int nb = (nRows + SKIP_ROWS - 1) / SKIP_ROWS;
  skip.assign(std::max(nb, 1), SdcSkip{(int32_t)hg.nOff, nRows, hg.offLen});
  if (hg.offType != CLA_OFF_BYTE && hg.offType != CLA_OFF_CHAR) return CLA_OK;
  const int maxV = hg.offType == CLA_OFF_BYTE ? 255 : 65535;
  const uint8_t* b = hg.offData.data();
  const uint16_t* c = (const uint16_t*)hg.offData.data();
  int64_t row = hg.first, elem = 0, pos = 0;
  int nextBlock = 0;
  auto note = [&](int64_t r, int64_t e, int64_t p) {
    while (nextBlock < nb && (int64_t)nextBlock * SKIP_ROWS <= r) skip[nextBlock++] = SdcSkip{(int32_t)e, (int32_t)r, p};
  };
  if (row < 0 || row >= nRows) return fail(CLA_ERR_BAD_ARG, "SDC offsetToFirst outside the matrix");
  note(row, 0, 0);
  while (pos < hg.offLen) {
    const int d = hg.offType == CLA_OFF_BYTE ? b[pos] : c[pos];
    pos++;
    if (d == 0) row += maxV;
    else {
      row += d;
      elem++;
      if (row >= nRows) return fail(CLA_ERR_BAD_ARG, "SDC offsets run past the last row");
      note(row, elem, pos);
    }
  }
  if (elem + 1 != hg.nOff) return fail(CLA_ERR_BAD_ARG, "SDC offset stream does not hold nOffsets rows");
  if (row != hg.last) return fail(CLA_ERR_BAD_ARG, "SDC offset stream does not end at offsetToLast");
  return CLA_OK;
}

int64_t init_device_state(Matrix* m) {
  CLA_CUDA(cudaSetDevice(m->device));
  cudaDeviceProp prop;
  CLA_CUDA(cudaGetDeviceProperties(&prop, m->device));
  m->smCount = prop.multiProcessorCount;
  CLA_CUDA(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
  CLA_CUDA(cudaEventCreate(&m->ev0));
  CLA_CUDA(cudaEventCreate(&m->ev1));
  CLA_CUDA(cudaEventCreateWithFlags(&m->lastDone, cudaEventDisableTiming));
  void* errp = nullptr;
  CLA_CUDA(cudaMalloc(&errp, 64));
  CLA_CUDA(cudaMemset(errp, 0, 64));
  m->dErr = (int32_t*)errp;
  return CLA_OK;
}

int64_t finalize_device(Matrix* m) {
  int64_t rc0 = init_device_state(m);
  if (rc0 < 0) return rc0;

  m->constV.assign(m->nCols, 0.0);
  m->regToDev.assign(m->hg.size(), -1);
  m->groups.clear();
  int64_t valOff = 0;
  m->colMin.assign(m->nCols, INFINITY);
  m->colMax.assign(m->nCols, -INFINITY);
  {
    std::vector<uint8_t> seen(m->nCols, 0);
    m->multiCover = false;
    for (auto& hg : m->hg)
      for (int c : hg.cols) {
        m->multiCover |= seen[c] != 0;
        seen[c] = 1;
      }
  }
  for (size_t gi = 0; gi < m->hg.size(); gi++) {
    HostGroup& hg = m->hg[gi];
    const int gc = (int)hg.cols.size();
    minmax_of_group(hg, m->nRows, m->colMin, m->colMax);
    if (hg.type == GT_EMPTY) continue;
    if (hg.type == GT_CONST) {  // ColGroupConst.addToCommon
      for (int j = 0; j < gc; j++) m->constV[hg.cols[j]] += hg.dict[j];
      continue;
    }
    DevGroup g;
    std::memset(&g, 0, sizeof(g));
    g.type = g.origType = hg.type;
    g.gCols = gc;
    g.nVals = hg.nVals;
    g.mapType = hg.mapType;
    g.mapSize = hg.mapSize;
    g.single = hg.single ? 1 : 0;
    int64_t rc;
    if ((rc = upload(m, hg.cols.data(), hg.cols.size(), &g.cols, true)) < 0) return rc;
    std::vector<double> dict = hg.dict;
    if (hg.type == GT_SDC && !hg.def.empty()) {  // extractCommon: default -> constV, dict -= default
      for (int j = 0; j < gc; j++) m->constV[hg.cols[j]] += hg.def[j];
      for (int k = 0; k < hg.nVals; k++)
        for (int j = 0; j < gc; j++) dict[(size_t)k * gc + j] -= hg.def[j];
    }
    if (hg.type == GT_OLE) {  // zero tuple behind the dictionary for rows that no value lists
      dict.resize((size_t)(hg.nVals + 1) * gc, 0.0);
      g.nVals = hg.nVals + 1;
    }
    if (hg.type != GT_UNC) {
      if ((rc = upload(m, dict.data(), dict.size(), &g.dict, true)) < 0) return rc;
      g.dictRaw = g.dict;
      // decompress of a non-overlapping block writes the registered values themselves, not (d - default) + default
      if (hg.type == GT_SDC && !hg.def.empty())
        if ((rc = upload(m, hg.dict.data(), hg.dict.size(), &g.dictRaw, true)) < 0) return rc;
    }

    if (hg.type == GT_DDC && hg.devMap) {  // registered from device memory: copy, then check the ids on the device
      size_t hiB;
      const size_t mb = map_bytes(hg.mapType, hg.mapSize, &hiB);
      uint8_t* dm = nullptr;
      if ((rc = dev_alloc(m, mb, &dm)) < 0) return rc;
      m->indexBytes += mb;
      if (hg.devSrcDevice == m->device || hg.devSrcDevice < 0)
        CLA_CUDA(cudaMemcpyAsync(dm, hg.devMap, mb, cudaMemcpyDeviceToDevice, m->stream));
      else
        CLA_CUDA(cudaMemcpyPeerAsync(dm, m->device, hg.devMap, hg.devSrcDevice, mb, m->stream));
      k_check_ids<<<grid_for(hg.mapSize, 256), 256, 0, m->stream>>>(hg.mapType, dm, hg.mapSize, hg.nVals, m->dErr);
      g.map = dm;
    } else if (hg.type == GT_DDC || hg.type == GT_SDC) {
      size_t hiB;
      const size_t mb = map_bytes(hg.mapType, hg.mapSize, &hiB);
      const uint8_t *dm = nullptr, *dh = nullptr;
      if ((rc = upload(m, hg.map.data(), mb, &dm, true)) < 0) return rc;
      if ((rc = upload(m, hg.mapHi.data(), hiB, &dh, true)) < 0) return rc;
      g.map = dm;
      g.mapHi = dh;
    }
    if (hg.type == GT_SDC) {
      g.offType = hg.offType;
      g.first = hg.first;
      g.last = hg.last;
      g.offLen = hg.offLen;
      g.nOff = hg.nOff;
      const uint8_t* od = nullptr;
      if ((rc = upload(m, hg.offData.data(), hg.offData.size(), &od, true)) < 0) return rc;
      g.offData = od;
      std::vector<SdcSkip> skip;
      if ((rc = build_sdc_skip(hg, m->nRows, skip)) < 0) return rc;
      if ((rc = upload(m, skip.data(), skip.size(), &g.skip, false)) < 0) return rc;
    }
    if (hg.type == GT_RLE || hg.type == GT_OLE) {
      if ((rc = upload(m, hg.ptr.data(), hg.ptr.size(), &g.ptr, true)) < 0) return rc;
      if ((rc = upload(m, hg.data.data(), hg.data.size(), &g.data, true)) < 0) return rc;
      g.dataLen = (int64_t)hg.data.size();
    }
    if (hg.type == GT_RLE) {
      if (hg.nVals >= 65535) return fail(CLA_ERR_UNSUPPORTED, "RLE group with 65535 or more values");
      const int64_t nPairs = (int64_t)hg.data.size() / 2;
      const int nb = (m->nRows + SKIP_ROWS - 1) / SKIP_ROWS;
      int32_t* dSkip = nullptr;
      if ((rc = dev_alloc(m, (size_t)std::max(nb, 1), &dSkip)) < 0) return rc;
      RleRun* dRuns = nullptr;
      if (nPairs > 0) {
        RleRun* tmpRuns = nullptr;
        uint32_t *k0 = nullptr, *k1 = nullptr, *v0 = nullptr, *v1 = nullptr;
        void* tmp = nullptr;
        CLA_CUDA(cudaMalloc(&tmp, nPairs * (sizeof(RleRun) + 4 * sizeof(uint32_t))));
        tmpRuns = (RleRun*)tmp;
        k0 = (uint32_t*)(tmpRuns + nPairs);
        k1 = k0 + nPairs;
        v0 = k1 + nPairs;
        v1 = v0 + nPairs;
        if ((rc = dev_alloc(m, (size_t)nPairs, &dRuns)) < 0) return rc;
        k_rle_decode<<<(hg.nVals * 32 + 255) / 256, 256, 0, m->stream>>>(g.ptr, g.data, hg.nVals, tmpRuns, k0, m->nRows,
                                                                        m->dErr);
        k_iota<<<(unsigned)((nPairs + 255) / 256), 256, 0, m->stream>>>(v0, nPairs);
        size_t tb = 0;
        cub::DeviceRadixSort::SortPairs(nullptr, tb, k0, k1, v0, v1, (int)nPairs, 0, 32, m->stream);
        void* dTmp = nullptr;
        CLA_CUDA(cudaMalloc(&dTmp, tb + 16));
        cub::DeviceRadixSort::SortPairs(dTmp, tb, k0, k1, v0, v1, (int)nPairs, 0, 32, m->stream);
        k_rle_gather<<<(unsigned)((nPairs + 255) / 256), 256, 0, m->stream>>>(tmpRuns, v1, dRuns, nPairs);
        // runs of length zero (the (65535, 0) fillers) sorted to the end: count the real ones on the host
        int64_t real = 0;
        for (int64_t i = 0; i < nPairs; i++) real += hg.data[2 * i + 1] != 0;
        g.nRuns = real;
        g.runs = dRuns;
        k_rle_skip<<<(nb + 255) / 256, 256, 0, m->stream>>>(dRuns, real, dSkip, nb);
        CLA_CUDA(cudaStreamSynchronize(m->stream));
        CLA_CUDA(cudaFree(dTmp));
        CLA_CUDA(cudaFree(tmp));
      } else {
        CLA_CUDA(cudaMemsetAsync(dSkip, 0, sizeof(int32_t) * std::max(nb, 1), m->stream));
      }
      g.runSkip = dSkip;
    }
    if (hg.type == GT_OLE) {  // transcode to a per-row map; products treat the group as DDC
      const int nv1 = hg.nVals + 1;
      const int64_t n = m->nRows;
      void* dm = nullptr;
      if (nv1 <= 256) {
        uint8_t* p;
        if ((rc = dev_alloc(m, (size_t)n, &p)) < 0) return rc;
        m->indexBytes += n;
        k_fill<uint8_t><<<grid_for(n, 256), 256, 0, m->stream>>>(p, (uint8_t)hg.nVals, n);
        if (hg.nVals) k_ole_to_map<uint8_t><<<(hg.nVals * 32 + 255) / 256, 256, 0, m->stream>>>(g.ptr, g.data, hg.nVals, p, (int)n, m->dErr);
        g.mapType = CLA_MAP_BYTE;
        dm = p;
      } else if (nv1 <= 65536) {
        uint16_t* p;
        if ((rc = dev_alloc(m, (size_t)n, &p)) < 0) return rc;
        m->indexBytes += n * 2;
        k_fill<uint16_t><<<grid_for(n, 256), 256, 0, m->stream>>>(p, (uint16_t)hg.nVals, n);
        k_ole_to_map<uint16_t><<<(hg.nVals * 32 + 255) / 256, 256, 0, m->stream>>>(g.ptr, g.data, hg.nVals, p, (int)n, m->dErr);
        g.mapType = CLA_MAP_CHAR;
        dm = p;
      } else {
        int32_t* p;
        if ((rc = dev_alloc(m, (size_t)n, &p)) < 0) return rc;
        m->indexBytes += n * 4;
        k_fill<int32_t><<<grid_for(n, 256), 256, 0, m->stream>>>(p, hg.nVals, n);
        k_ole_to_map<int32_t><<<(hg.nVals * 32 + 255) / 256, 256, 0, m->stream>>>(g.ptr, g.data, hg.nVals, p, (int)n, m->dErr);
        g.mapType = CLA_MAP_INT;
        dm = p;
      }
      g.map = dm;
      g.mapSize = n;
      g.type = GT_DDC;
    }
    if (hg.type == GT_UNC && hg.devDense) {
      double* dd = nullptr;
      const size_t n = (size_t)m->nRows * gc;
      if ((rc = dev_alloc(m, n, &dd)) < 0) return rc;
      m->indexBytes += n * sizeof(double);
      if (hg.devSrcDevice == m->device || hg.devSrcDevice < 0)
        CLA_CUDA(cudaMemcpyAsync(dd, hg.devDense, n * sizeof(double), cudaMemcpyDeviceToDevice, m->stream));
      else
        CLA_CUDA(cudaMemcpyPeerAsync(dd, m->device, hg.devDense, hg.devSrcDevice, n * sizeof(double), m->stream));
      g.dense = dd;
    } else if (hg.type == GT_UNC) {
      if ((rc = upload(m, hg.dense.data(), hg.dense.size(), &g.dense, true)) < 0) return rc;
    } else {
      g.valOff = valOff;
      valOff += g.nVals;
    }
    m->regToDev[gi] = (int)m->groups.size();
    m->groups.push_back(g);
  }
  m->totalVals = valOff;
  m->nDev = (int)m->groups.size();
  m->hasConst = false;
  for (double x : m->constV) m->hasConst |= (x != 0.0);
  CLA_CUDA(cudaStreamSynchronize(m->stream));
  int32_t herr = 0;
  CLA_CUDA(cudaMemcpy(&herr, m->dErr, sizeof(herr), cudaMemcpyDeviceToHost));
  if (herr) {
    cudaMemset(m->dErr, 0, sizeof(int32_t));
    return fail(herr == 3 ? CLA_ERR_BAD_ARG : CLA_ERR_DEVICE_CHECK,
                herr == 1 ? "RLE run past the last row"
                          : (herr == 3 ? "device-resident map holds an id at or above the number of dictionary tuples"
                                       : "OLE offset past the last row"));
  }
  const DevGroup* dg = nullptr;
  int64_t rc;
  if ((rc = upload(m, m->groups.data(), m->groups.size(), &dg, false)) < 0) return rc;
  m->dGroups = const_cast<DevGroup*>(dg);
  const double* dc = nullptr;
  if ((rc = upload(m, m->constV.data(), m->constV.size(), &dc, false)) < 0) return rc;
  m->dConstV = const_cast<double*>(dc);
  {  // column -> (group, position); valid when no column is held by two product groups (decompress, fused TSMM)
    std::vector<int32_t> colSrc((size_t)m->nCols * 2, -1);
    m->colSrcValid = true;
    for (size_t gi = 0; gi < m->hg.size(); gi++) {
      if (m->regToDev[gi] < 0) continue;
      const DevGroup& g = m->groups[m->regToDev[gi]];
      for (int j = 0; j < g.gCols; j++) {  // every product group: dense-map, uncompressed, SDC, RLE
        const int c = m->hg[gi].cols[j];
        if (colSrc[2 * c] >= 0) m->colSrcValid = false;
        colSrc[2 * c] = m->regToDev[gi];
        colSrc[2 * c + 1] = j;
      }
    }
    const int32_t* dcs = nullptr;
    if ((rc = upload(m, colSrc.data(), colSrc.size(), &dcs, false)) < 0) return rc;
    m->dColSrc = const_cast<int32_t*>(dcs);
  }
  // the registered host arrays are no longer needed
  for (auto& hg : m->hg) {
    std::vector<uint8_t>().swap(hg.map);
    std::vector<uint8_t>().swap(hg.mapHi);
    std::vector<uint8_t>().swap(hg.offData);
    std::vector<uint16_t>().swap(hg.data);
    std::vector<double>().swap(hg.dense);
  }
  if ((rc = fast_plan_build(m)) < 0) return rc;
  m->stats.n_rows = m->nRows;
  m->stats.n_cols = m->nCols;
  m->stats.n_groups = (int64_t)m->hg.size();
  m->stats.device_bytes = m->deviceBytes;
  m->stats.index_bytes = m->indexBytes;
  m->finalized = true;
  return CLA_OK;
}

void release(Matrix* m) {
  if (m->device >= 0) cudaSetDevice(m->device);
  fast_plan_free(m);
  for (void* p : m->allocs) cudaFree(p);
  m->allocs.clear();
  if (m->scratch) cudaFree(m->scratch);
  if (m->scratch2) cudaFree(m->scratch2);
  if (m->io) cudaFree(m->io);
  if (m->small_) cudaFree(m->small_);
  m->small_ = nullptr;
  if (m->dErr) cudaFree(m->dErr);
  for (auto& pr : m->profEvents) {
    cudaEventDestroy(pr.first);
    cudaEventDestroy(pr.second);
  }
  m->profEvents.clear();
  if (m->ev0) cudaEventDestroy(m->ev0);
  if (m->ev1) cudaEventDestroy(m->ev1);
  if (m->lastDone) cudaEventDestroy(m->lastDone);
  m->lastDone = nullptr;
  m->lastValid = false;
  for (auto& e : m->copyDone)
    if (e) {
      cudaEventDestroy(e);
      e = nullptr;
    }
  if (m->copyStream) cudaStreamDestroy(m->copyStream);
  m->copyStream = nullptr;
  host_stage_free(m);
  if (m->stream) cudaStreamDestroy(m->stream);
  m->scratch = m->scratch2 = m->io = nullptr;
  m->dErr = nullptr;
  m->stream = nullptr;
}

cla_handle table_insert(std::shared_ptr<Matrix> m) {
  std::lock_guard<std::mutex> lk(g_tabMu);
  const int64_t h = g_next++;
  g_table[h] = std::move(m);
  return h;
}
bool table_erase(cla_handle h, std::shared_ptr<Matrix>* out) {
  std::lock_guard<std::mutex> lk(g_tabMu);
  auto it = g_table.find(h);
  if (it == g_table.end()) return false;
  *out = it->second;
  g_table.erase(it);
  return true;
}

}  // namespace cla
