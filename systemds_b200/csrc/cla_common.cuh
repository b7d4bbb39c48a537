// Shared declarations of the CLA device library: device-side group records, the host-side
// matrix object behind a cla_handle, and helpers used by every translation unit.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <memory>
#include <functional>
#include <mutex>
#include <string>
#include <vector>
#include "../../include/systemds_cla.h"

namespace cla {

constexpr int SKIP_ROWS = 1024;  // granularity of the SDC / RLE skip indexes (AOffset's skip list uses ~1000)
constexpr int BITMAP_BLOCK_SZ = 65535;

enum GroupType : int { GT_DDC = 0, GT_SDC = 1, GT_RLE = 2, GT_OLE = 3, GT_UNC = 4, GT_CONST = 5, GT_EMPTY = 6 };

// Start state for decoding an offset stream at a row-block boundary: the first listed row at or
// after the boundary, its position in the map (AIterator.getDataIndex), and the stream position
// right behind it.
struct SdcSkip {
  int32_t elem;  // index of that element (== nOff when there is none)
  int32_t row;   // its row
  int64_t pos;   // index of the next delta to read
};

// One run of a value, in absolute rows (decoded from the (gap, len) pairs and merged over values).
struct RleRun {
  int32_t start;
  uint16_t len;
  uint16_t k;
};

// Device-visible record of one column group. All pointers are device addresses.
struct DevGroup {
  int32_t type;      // how products treat it: GT_DDC (also transcoded OLE), GT_SDC, GT_RLE, GT_UNC
  int32_t origType;  // the registered type
  int32_t gCols, nVals;
  int32_t mapType;
  int32_t single;  // SDCSingle*: every listed row holds tuple 0
  int32_t offType, first, last;
  int32_t inFast;  // 1: the specialised vector kernels cover this group (general kernels skip it on their request)
  int64_t mapSize, offLen, nOff, nRuns, dataLen;
  int64_t valOff;  // first row of this group's table in the per-call value arenas (sum of nVals before it)
  const int32_t* cols;
  const double* dict;  // effective dictionary (default tuple subtracted), [nVals x gCols]
  const double* dictRaw;  // the dictionary as registered (== dict unless a default tuple was folded into constV)
  const void* map;
  const void* mapHi;
  const void* offData;
  const SdcSkip* skip;
  const RleRun* runs;
  const int32_t* runSkip;  // per SKIP_ROWS block: first run whose end lies behind the block start
  const int32_t* ptr;      // RLE / OLE as registered
  const uint16_t* data;
  const double* dense;  // UNC [nRows x gCols]
};

// Read one cell of a map in the reference's storage layout.
__device__ __forceinline__ int map_get(int mapType, const void* __restrict__ map, const void* __restrict__ mapHi,
                                       int64_t r) {
  switch (mapType) {
    case CLA_MAP_ZERO: return 0;
    case CLA_MAP_BIT: return (int)((((const unsigned long long*)map)[r >> 6] >> (r & 63)) & 1ULL);
    case CLA_MAP_UBYTE:
    case CLA_MAP_BYTE: return ((const uint8_t*)map)[r];
    case CLA_MAP_CHAR: return ((const uint16_t*)map)[r];
    case CLA_MAP_CHAR_BYTE: return (int)((const uint16_t*)map)[r] + ((int)((const uint8_t*)mapHi)[r] << 16);
    default: return ((const int32_t*)map)[r];
  }
}

// Warp-level decode of one SKIP_ROWS block of an offset stream: deltas are read 32 at a time,
// a warp scan turns them into rows, a ballot numbers the elements (continuation deltas carry none).
// f(row, elemIndex) is called for every listed row in [rowBegin, rowEnd).
template <class F>
__device__ __forceinline__ void sdc_walk_block(const DevGroup& g, int rowBegin, int rowEnd, F&& f) {
  const int lane = threadIdx.x & 31;
  if (g.nOff == 0) return;
  if (g.offType == CLA_OFF_SINGLE || g.offType == CLA_OFF_TWO) {
    if (lane == 0) {
      if (g.first >= rowBegin && g.first < rowEnd) f(g.first, 0);
      if (g.offType == CLA_OFF_TWO && g.last >= rowBegin && g.last < rowEnd) f(g.last, 1);
    }
    return;
  }
  const SdcSkip sk = g.skip[rowBegin / SKIP_ROWS];
  int row = sk.row;
  int elem = sk.elem;
  int64_t pos = sk.pos;
  if (elem >= g.nOff || row >= rowEnd) return;
  if (lane == 0 && row >= rowBegin) f(row, elem);
  const int maxV = g.offType == CLA_OFF_BYTE ? 255 : 65535;
  while (pos < g.offLen) {
    const int64_t i = pos + lane;
    int d = 0;
    if (i < g.offLen) d = g.offType == CLA_OFF_BYTE ? (int)((const uint8_t*)g.offData)[i] : (int)((const uint16_t*)g.offData)[i];
    const bool inb = i < g.offLen;
    int inc = inb ? (d == 0 ? maxV : d) : 0;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, inc, s);
      if (lane >= s) inc += t;
    }
    const bool isElem = inb && d != 0;
    const unsigned bal = __ballot_sync(0xffffffffu, isElem);
    const int myRow = row + inc;
    const int myElem = elem + __popc(bal & ((2u << lane) - 1u));
    if (isElem && myRow >= rowBegin && myRow < rowEnd) f(myRow, myElem);
    row += __shfl_sync(0xffffffffu, inc, 31);
    elem += __popc(bal);
    pos += 32;
    if (row >= rowEnd) break;
  }
}

// Host-side group as registered (arrays copied from the caller).
struct HostGroup {
  int type = GT_DDC;
  std::vector<int32_t> cols;
  int nVals = 0;
  std::vector<double> dict;
  std::vector<double> def;  // default tuple (empty = zeros)
  int mapType = CLA_MAP_ZERO;
  int64_t mapSize = 0;
  std::vector<uint8_t> map, mapHi;  // raw bytes
  bool single = false;
  int offType = CLA_OFF_EMPTY, first = 0, last = 0;
  int64_t offLen = 0, nOff = 0;
  std::vector<uint8_t> offData;
  std::vector<int32_t> ptr;
  std::vector<uint16_t> data;
  std::vector<double> dense;
  // Groups registered from device memory (cla_add_group_ddc_dev / cla_add_group_uncompressed_dev): the caller's
  // buffer, read once at cla_finalize and copied device to device.
  const void* devMap = nullptr;
  const double* devDense = nullptr;
  int devSrcDevice = -1;
};

// Row-major work lists of the SDC / RLE groups (built by ensure_sparse_lists, cla_rmm_dmma.cu): rows are cut into
// steps of 8 and windows of 64, a warp work unit of the tensor-core right product is 512 rows.
constexpr int G3_UNIT = 512;
constexpr int G3_STEP = 8;
constexpr int G3_WIN = 64;
// One piece of work: rows [ra, rb) of an 8-row step (or a whole 64-row window) receive table row prow.
struct SpItem {
  uint32_t prow;
  uint32_t rows;  // ra | rb << 8 | (index of the step or window inside its 1024-row block) << 16
};

struct FastPlan;  // plans of the specialised DDC kernels (cla_fast.cu)
struct HostStage; // pinned ring for operands in pageable host memory (cla_hostcopy.cu)

struct Matrix;
struct Matrix {
  // A block returned by cla_rmm_overlapping shares the index structures of the block it was computed from; it
  // keeps that block alive (parent), and a parent destroyed before its children only leaves the handle table: its
  // device memory is released with the last child (children, zombie; both guarded by the parent's mutex).
  std::shared_ptr<Matrix> parent;
  int children = 0;
  bool zombie = false;
  int32_t nRows = 0, nCols = 0;
  bool overlapping = false;
  bool finalized = false;
  int device = -1;
  std::mutex mu;
  std::vector<HostGroup> hg;   // cleared after finalize (records kept, arrays dropped)
  std::vector<DevGroup> groups;  // host copy of the device records (product groups only)
  std::vector<int> regToDev;     // registered group index -> index in groups (-1: const / empty)
  DevGroup* dGroups = nullptr;
  int nDev = 0;
  int64_t totalVals = 0;         // sum of nVals over dictionary groups
  std::vector<double> constV;    // host copy
  std::vector<double> colMin, colMax;  // per-column extrema over the compressed groups, dictionary-based (cla_agg.cu)
  bool multiCover = false;             // some column is held by more than one registered group (e.g. FOR group + reference)
  double* dConstV = nullptr;     // [nCols]
  void* dDenseCols = nullptr;    // list of dense-operand columns for the tensor-core RMM (built on first use)
  int nDenseCols = 0;
  void* dDenseDesc = nullptr;    // the same columns as flat records (map, dictionary column, V row)
  void* dSdcIdx = nullptr;       // device group indices of the SDC / RLE groups
  void* dRleIdx = nullptr;
  int nSdcGroups = 0, nRleGroups = 0;
  bool denseColsBuilt = false;
  int32_t* dSparseIdx = nullptr;  // device group indices of the SDC groups with listed rows and RLE groups with runs, list order
  int nSparse = 0;
  // the other groups by kind, list order: dense-map groups (all, then those the specialised kernels do not take), uncompressed
  int32_t* dDdcIdx = nullptr;
  int32_t* dDdcRestIdx = nullptr;
  int32_t* dUncIdx = nullptr;
  int nDdc = 0, nDdcRest = 0, nUnc = 0;
  bool sparseListBuilt = false;
  // row-major work lists of the SDC / RLE groups for the tensor-core right product (cla_rmm_dmma.cu), built on first use
  void* dStepItems = nullptr;
  uint32_t* dStepPtr = nullptr;
  void* dWinItems = nullptr;
  uint32_t* dWinPtr = nullptr;
  bool spListsTried = false, spListsOk = false;
  int64_t nStepPtr = 0, nWinPtr = 0;  // entries of dStepPtr / dWinPtr (the last one = number of items)
  int32_t* dColSrc = nullptr;    // [nCols][2]: dense-map / uncompressed group holding the column and the position in it (-1: none)
  bool colSrcValid = false;      // false when some column is held by more than one such group (overlapping input)
  bool hasConst = false;
  std::vector<void*> allocs;     // everything cudaMalloc'ed for the groups
  int64_t deviceBytes = 0, indexBytes = 0;
  // growable scratch (value arenas, partial results, host staging)
  void* scratch = nullptr;
  size_t scratchBytes = 0;
  void* scratch2 = nullptr;
  size_t scratch2Bytes = 0;
  void* small_ = nullptr;  // small per-call vectors (row sums of the left operand)
  size_t smallBytes = 0;
  void* io = nullptr;  // device staging for host-buffer calls
  size_t ioBytes = 0;
  int32_t* dErr = nullptr;  // device self-check word
  cudaStream_t stream = nullptr;
  cudaStream_t copyStream = nullptr;  // uploads overlapped with kernels in the host-buffer left product
  cudaEvent_t copyDone[16] = {};  // one per row range of the pipelined host-buffer left product
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  // Every product call uses the handle's one set of scratch buffers. A call that arrives on another stream than
  // the previous one first waits for `lastDone` (recorded when the previous call had enqueued its work), so two
  // calls on one handle never overlap on the GPU even when their streams would allow it.
  cudaEvent_t lastDone = nullptr;
  cudaStream_t lastStream = nullptr;
  bool lastValid = false;
  FastPlan* fast = nullptr;
  HostStage* hostStage = nullptr;
  bool profile = false;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> profEvents;  // ring of event pairs
  size_t profUsed = 0;
  cla_stats stats{};
  int smCount = 148;
};

// error plumbing --------------------------------------------------------------------------------
void set_error(const std::string& msg);
int64_t fail(int64_t code, const std::string& msg);
#define CLA_CUDA(expr)                                                                              \
  do {                                                                                              \
    cudaError_t e_ = (expr);                                                                        \
    if (e_ != cudaSuccess)                                                                          \
      return ::cla::fail(CLA_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e_));         \
  } while (0)

// profiling brackets around the dominant kernel of a product call (no-ops unless m->profile)
void prof_begin(Matrix* m, cudaStream_t s);
void prof_end(Matrix* m, cudaStream_t s);
void prof_collect(Matrix* m);

int64_t order_begin(Matrix* m, cudaStream_t s);  // see Matrix::lastDone
int64_t order_end(Matrix* m, cudaStream_t s);
int64_t ensure_scratch(Matrix* m, size_t bytes);
int64_t ensure_scratch2(Matrix* m, size_t bytes);
int64_t ensure_io(Matrix* m, size_t bytes);
int64_t ensure_small(Matrix* m, size_t bytes);
// Transfers between pageable host memory and the device through the handle's pinned ring (cla_hostcopy.cu).
// host_copy_staged: whether a transfer of `bytes` at `host` should take them (large, pageable, ring available).
bool host_copy_staged(Matrix* m, const void* host, size_t bytes);
int64_t host_to_device_staged(Matrix* m, void* dDst, const void* host, size_t bytes, cudaStream_t cs,
                              const std::function<int64_t(size_t)>& enqueued);
int64_t device_to_host_staged(Matrix* m, void* host, const void* dSrc, size_t bytes, cudaStream_t s);
void host_stage_free(Matrix* m);
int64_t ensure_sparse_list(Matrix* m);
int64_t ensure_sparse_lists(Matrix* m, cudaStream_t s);  // the row-major work lists; m->spListsOk tells whether they exist  // Matrix::dSparseIdx (cla_generic.cu)

// launchers implemented in the kernel translation units; all enqueue on `s` and return CLA_OK or an error.
int64_t launch_rmm(Matrix* m, const double* dV, int vCols, double* dOut, cudaStream_t s, bool afterFast = false);
int64_t launch_rmm_dmma(Matrix* m, const double* dV, int vCols, double* dOut, cudaStream_t s);
int64_t launch_lmm(Matrix* m, const double* dYt, int q, double* dOut, cudaStream_t s, bool afterFast = false);
void minmax_of_group(const HostGroup& hg, int nRows, std::vector<double>& colMin, std::vector<double>& colMax);
int64_t col_minmax(Matrix* m, std::vector<double>& lo, std::vector<double>& hi, cudaStream_t s);
int64_t row_minmax(Matrix* m, int wantMax, double* dOut, cudaStream_t s);
int64_t launch_tsmm(Matrix* m, double* dOut, cudaStream_t s);
int64_t launch_tmm(Matrix* left, Matrix* right, double* dOut, cudaStream_t s);  // t(left) %*% right, both compressed
// products on the dictionaries of two all-dense-map operands (cla_pairs.cu)
bool pairs_eligible(const Matrix* L, const Matrix* R, bool self);
int64_t launch_pairs(Matrix* L, Matrix* R, bool self, double* dOut, cudaStream_t s);
int64_t launch_decompress(Matrix* m, double* dOut, cudaStream_t s);
// X %*% V kept compressed: fills `child` (fresh Matrix) with groups that alias m's index structures (cla_generic.cu)
int64_t make_overlapping(Matrix* m, Matrix* child, const double* dV, int vCols, cudaStream_t s);
int64_t init_device_state(Matrix* m);  // stream, events, error word of a Matrix whose device is set (cla_finalize.cu)
int64_t launch_decompress_range(Matrix* m, int r0, int r1, double* dOut, cudaStream_t s);
int64_t launch_group_decode(Matrix* m, int devGroup, int32_t* dIds, cudaStream_t s);
int64_t launch_group_counts(Matrix* m, int devGroup, unsigned long long* dCounts, cudaStream_t s);
int64_t launch_count_nnz(Matrix* m, const double* d, int64_t n, unsigned long long* dCount, cudaStream_t s);
int64_t launch_scale_rows(Matrix* m, double* dU, const double* dW, int64_t n, cudaStream_t s);

// finalize-time device work (cla_finalize.cu)
int64_t finalize_device(Matrix* m);
// fast paths (cla_fast.cu): return 1 if they handled the whole product, 2 if they handled the groups marked inFast
// (the caller then runs the general launcher with afterFast = true), 0 if not applicable, <0 on error
int64_t fast_plan_build(Matrix* m);
void fast_plan_free(Matrix* m);
bool fast_plan_ok(const Matrix* m);       // some or all groups are covered by the specialised kernels
bool fast_plan_partial(const Matrix* m);  // ... some but not all
int64_t fast_rmm_vec(Matrix* m, const double* dV, double* dOut, cudaStream_t s);
int64_t fast_lmm_vec(Matrix* m, const double* dY, double* dOut, cudaStream_t s);
int64_t fast_lmm_rows(Matrix* m, const double* dY, size_t pitch, int q, double* dOut, cudaStream_t s);  // q = 2 or 4 left rows at once
int64_t fast_decompress(Matrix* m, int r0, int r1, double* dOut, cudaStream_t s);  // 1 = done, 0 = not covered
int64_t fast_lmm_vec_host(Matrix* m, const double* hostY, double* dY, double* dOut, cudaStream_t s);
int64_t fast_lmm_vec_noalloc(Matrix* m, const double* dY, double* dOut, cudaStream_t s);

}  // namespace cla
