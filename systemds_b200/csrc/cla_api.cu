// extern "C" entry points declared in include/systemds_cla.h.
#include "cla_common.cuh"
#include <cmath>
#include <cstring>
#include <memory>
#include <vector>

namespace cla {
int64_t measure_fp64_peaks(int device, double* dmmaTflops, double* dfmaTflops);
std::shared_ptr<Matrix> lookup(cla_handle h);
cla_handle table_insert(std::shared_ptr<Matrix> m);
bool table_erase(cla_handle h, std::shared_ptr<Matrix>* out);
void release(Matrix* m);
const std::string& last_error();
}  // namespace cla

using namespace cla;

#define GET_MATRIX(h)                                                       \
  std::shared_ptr<Matrix> mp = lookup(h);                                   \
  if (!mp) return fail(CLA_ERR_BAD_HANDLE, "unknown or destroyed handle");  \
  Matrix* m = mp.get();                                                     \
  std::lock_guard<std::mutex> lk(m->mu)

#define REQUIRE_OPEN()  \
  if (m->finalized) return fail(CLA_ERR_STATE, "groups cannot be added after cla_finalize")
#define REQUIRE_FINAL() \
  if (!m->finalized) return fail(CLA_ERR_STATE, "cla_finalize has not been called on this handle")

static int64_t check_cols(Matrix* m, const int32_t* colIdx, int32_t gCols) {
  if (!colIdx || gCols <= 0) return fail(CLA_ERR_BAD_ARG, "group needs at least one column index");
  for (int j = 0; j < gCols; j++)
    if (colIdx[j] < 0 || colIdx[j] >= m->nCols) return fail(CLA_ERR_SHAPE, "column index outside the matrix");
  return CLA_OK;
}

static size_t map_raw_bytes(int mapType, int64_t size, size_t* hi) {
  *hi = 0;
  switch (mapType) {
    case CLA_MAP_ZERO: return 0;
    case CLA_MAP_BIT: return (size_t)((size + 63) / 64) * 8;
    case CLA_MAP_UBYTE:
    case CLA_MAP_BYTE: return (size_t)size;
    case CLA_MAP_CHAR: return (size_t)size * 2;
    case CLA_MAP_CHAR_BYTE: *hi = (size_t)size; return (size_t)size * 2;
    case CLA_MAP_INT: return (size_t)size * 4;
    default: return 0;
  }
}

// Ids must stay below nVals: the kernels index dictionaries with them unchecked.
static int64_t check_map(int mapType, const uint8_t* map, const uint8_t* hi, int64_t size, int nVals) {
  int64_t mx = 0;
  switch (mapType) {
    case CLA_MAP_ZERO: mx = 0; break;
    case CLA_MAP_BIT: {
      const uint64_t* w = (const uint64_t*)map;
      uint64_t any = 0;
      for (int64_t i = 0; i < (size + 63) / 64; i++) any |= w[i];
      mx = any ? 1 : 0;
      break;
    }
    case CLA_MAP_UBYTE:
    case CLA_MAP_BYTE:
      for (int64_t i = 0; i < size; i++) mx = map[i] > mx ? map[i] : mx;
      break;
    case CLA_MAP_CHAR: {
      const uint16_t* c = (const uint16_t*)map;
      for (int64_t i = 0; i < size; i++) mx = c[i] > mx ? c[i] : mx;
      break;
    }
    case CLA_MAP_CHAR_BYTE: {
      const uint16_t* c = (const uint16_t*)map;
      for (int64_t i = 0; i < size; i++) {
        int64_t v = (int64_t)c[i] + ((int64_t)hi[i] << 16);
        mx = v > mx ? v : mx;
      }
      break;
    }
    case CLA_MAP_INT: {
      const int32_t* c = (const int32_t*)map;
      for (int64_t i = 0; i < size; i++) {
        if (c[i] < 0) return fail(CLA_ERR_BAD_ARG, "negative id in map");
        mx = c[i] > mx ? c[i] : mx;
      }
      break;
    }
    default: return fail(CLA_ERR_BAD_ARG, "unknown map type");
  }
  if (size > 0 && mx >= nVals) return fail(CLA_ERR_BAD_ARG, "map holds an id at or above the number of dictionary tuples");
  return CLA_OK;
}

static int64_t check_errword(Matrix* m);

extern "C" {

cla_handle cla_create(int32_t nRows, int32_t nCols, int32_t overlapping) {
  if (nRows < 0 || nCols < 0) return fail(CLA_ERR_BAD_ARG, "negative matrix dimension");
  auto m = std::make_shared<Matrix>();
  m->nRows = nRows;
  m->nCols = nCols;
  m->overlapping = overlapping != 0;
  return table_insert(m);
}

int64_t cla_destroy(cla_handle h) {
  std::shared_ptr<Matrix> mp;
  if (!table_erase(h, &mp)) return fail(CLA_ERR_BAD_HANDLE, "unknown or destroyed handle");
  std::shared_ptr<Matrix> parent;
  {
    std::lock_guard<std::mutex> lk(mp->mu);
    if (mp->children > 0) {  // blocks from cla_rmm_overlapping still read this one's index structures
      mp->zombie = true;
      return CLA_OK;
    }
    release(mp.get());
    parent = std::move(mp->parent);
  }
  while (parent) {  // the last child of a destroyed parent frees it too
    std::shared_ptr<Matrix> next;
    {
      std::lock_guard<std::mutex> lk(parent->mu);
      if (--parent->children > 0 || !parent->zombie) break;
      release(parent.get());
      next = std::move(parent->parent);
    }
    parent = std::move(next);
  }
  return CLA_OK;
}

int64_t cla_last_error(char* buf, int64_t cap) {
  const std::string& e = last_error();
  if (buf && cap > 0) {
    const size_t n = std::min<size_t>(e.size(), (size_t)cap - 1);
    std::memcpy(buf, e.data(), n);
    buf[n] = 0;
  }
  return (int64_t)e.size();
}

int64_t cla_stats_get(cla_handle h, cla_stats* out) {
  GET_MATRIX(h);
  if (!out) return fail(CLA_ERR_BAD_ARG, "null stats pointer");
  if (m->device >= 0) cudaSetDevice(m->device);
  prof_collect(m);
  if (m->finalized) {  // device-buffer calls do not synchronise: this is where their kernels' self-checks surface
    int64_t rc = check_errword(m);
    if (rc < 0) return rc;
  }
  *out = m->stats;
  out->n_rows = m->nRows;
  out->n_cols = m->nCols;
  out->n_groups = (int64_t)m->hg.size();
  return CLA_OK;
}

int64_t cla_measure_fp64_peaks(int32_t device, double* dmmaTflops, double* dfmaTflops) {
  if (!dmmaTflops || !dfmaTflops) return fail(CLA_ERR_BAD_ARG, "null output");
  return measure_fp64_peaks(device, dmmaTflops, dfmaTflops);
}

int64_t cla_set_profile(cla_handle h, int32_t on) {
  GET_MATRIX(h);
  m->profile = on != 0;
  return CLA_OK;
}

static int64_t add_dict_group(Matrix* m, HostGroup& g, int type, const int32_t* colIdx, int32_t gCols,
                              const double* dict, int32_t nVals) {
  int64_t rc = check_cols(m, colIdx, gCols);
  if (rc < 0) return rc;
  if (nVals < 0 || (nVals > 0 && !dict)) return fail(CLA_ERR_BAD_ARG, "dictionary missing");
  g.type = type;
  g.cols.assign(colIdx, colIdx + gCols);
  g.nVals = nVals;
  if (nVals) g.dict.assign(dict, dict + (size_t)nVals * gCols);
  return CLA_OK;
}

int64_t cla_add_group_ddc(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dict, int32_t nVals,
                          int32_t mapType, const void* map, const void* mapHi, int64_t mapSize) {
  GET_MATRIX(h);
  REQUIRE_OPEN();
  HostGroup g;
  int64_t rc = add_dict_group(m, g, GT_DDC, colIdx, gCols, dict, nVals);
  if (rc < 0) return rc;
  if (mapSize != m->nRows) return fail(CLA_ERR_SHAPE, "DDC map must have one cell per row");
  if (m->nRows > 0 && nVals == 0) return fail(CLA_ERR_BAD_ARG, "DDC group without dictionary tuples");
  size_t hi;
  const size_t mb = map_raw_bytes(mapType, mapSize, &hi);
  if ((mb && !map) || (hi && !mapHi)) return fail(CLA_ERR_BAD_ARG, "map array missing");
  if ((rc = check_map(mapType, (const uint8_t*)map, (const uint8_t*)mapHi, mapSize, nVals)) < 0) return rc;
  g.mapType = mapType;
  g.mapSize = mapSize;
  if (mb) g.map.assign((const uint8_t*)map, (const uint8_t*)map + mb);
  if (hi) g.mapHi.assign((const uint8_t*)mapHi, (const uint8_t*)mapHi + hi);
  m->hg.push_back(std::move(g));
  return (int64_t)m->hg.size() - 1;
}

int64_t cla_add_group_sdc(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dict, int32_t nVals,
                          const double* defaultTuple, int32_t offType, int32_t offsetToFirst, int32_t offsetToLast,
                          const void* offData, int64_t offLen, int64_t nOffsets, int32_t mapType, const void* map,
                          const void* mapHi) {
  GET_MATRIX(h);
  REQUIRE_OPEN();
  HostGroup g;
  int64_t rc = add_dict_group(m, g, GT_SDC, colIdx, gCols, dict, nVals);
  if (rc < 0) return rc;
  if (offType < CLA_OFF_EMPTY || offType > CLA_OFF_CHAR) return fail(CLA_ERR_BAD_ARG, "unknown offset type");
  if (nOffsets < 0 || nOffsets > m->nRows) return fail(CLA_ERR_SHAPE, "more offsets than rows");
  if (offType == CLA_OFF_EMPTY && nOffsets != 0) return fail(CLA_ERR_BAD_ARG, "empty offsets with a size");
  if (offType == CLA_OFF_SINGLE && nOffsets != 1) return fail(CLA_ERR_BAD_ARG, "OffsetSingle holds one row");
  if (offType == CLA_OFF_TWO && nOffsets != 2) return fail(CLA_ERR_BAD_ARG, "OffsetTwo holds two rows");
  if (nOffsets > 0 && (offsetToFirst < 0 || offsetToLast >= m->nRows || offsetToFirst > offsetToLast))
    return fail(CLA_ERR_SHAPE, "offsets outside the matrix");
  if ((offType == CLA_OFF_BYTE || offType == CLA_OFF_CHAR) && offLen > 0 && !offData)
    return fail(CLA_ERR_BAD_ARG, "offset array missing");
  if (nOffsets > 0 && nVals == 0) return fail(CLA_ERR_BAD_ARG, "SDC group without dictionary tuples");
  if (defaultTuple) g.def.assign(defaultTuple, defaultTuple + gCols);
  g.offType = offType;
  g.first = offsetToFirst;
  g.last = offsetToLast;
  g.nOff = nOffsets;
  if (offType == CLA_OFF_BYTE || offType == CLA_OFF_CHAR) {
    g.offLen = offLen;
    const size_t ob = (size_t)offLen * (offType == CLA_OFF_BYTE ? 1 : 2);
    if (ob) g.offData.assign((const uint8_t*)offData, (const uint8_t*)offData + ob);
  }
  g.single = (map == nullptr);
  if (!g.single) {
    size_t hi;
    const size_t mb = map_raw_bytes(mapType, nOffsets, &hi);
    if (hi && !mapHi) return fail(CLA_ERR_BAD_ARG, "map array missing");
    if ((rc = check_map(mapType, (const uint8_t*)map, (const uint8_t*)mapHi, nOffsets, nVals)) < 0) return rc;
    g.mapType = mapType;
    g.mapSize = nOffsets;
    if (mb) g.map.assign((const uint8_t*)map, (const uint8_t*)map + mb);
    if (hi) g.mapHi.assign((const uint8_t*)mapHi, (const uint8_t*)mapHi + hi);
  } else {
    g.mapType = CLA_MAP_ZERO;
    g.mapSize = nOffsets;
  }
  m->hg.push_back(std::move(g));
  return (int64_t)m->hg.size() - 1;
}

static int64_t add_offset_group(cla_handle h, int type, const int32_t* colIdx, int32_t gCols, const double* dict,
                                int32_t nVals, const int32_t* ptr, const uint16_t* data, int64_t dataLen) {
  GET_MATRIX(h);
  REQUIRE_OPEN();
  HostGroup g;
  int64_t rc = add_dict_group(m, g, type, colIdx, gCols, dict, nVals);
  if (rc < 0) return rc;
  if (!ptr) return fail(CLA_ERR_BAD_ARG, "_ptr array missing");
  if (dataLen < 0 || (dataLen > 0 && !data)) return fail(CLA_ERR_BAD_ARG, "_data array missing");
  if (ptr[0] != 0 || ptr[nVals] != dataLen) return fail(CLA_ERR_BAD_ARG, "_ptr does not span _data");
  for (int k = 0; k < nVals; k++)
    if (ptr[k + 1] < ptr[k] || (type == GT_RLE && ((ptr[k + 1] - ptr[k]) & 1)))
      return fail(CLA_ERR_BAD_ARG, "_ptr not monotone (or an RLE list of odd length)");
  if (type == GT_OLE)
    for (int k = 0; k < nVals; k++) {  // segment headers must chain exactly to the end of the list
      int64_t bix = ptr[k];
      while (bix < ptr[k + 1]) bix += (int64_t)data[bix] + 1;
      if (bix != ptr[k + 1]) return fail(CLA_ERR_BAD_ARG, "OLE segment headers do not chain to the list end");
    }
  g.ptr.assign(ptr, ptr + nVals + 1);
  if (dataLen) g.data.assign(data, data + dataLen);
  m->hg.push_back(std::move(g));
  return (int64_t)m->hg.size() - 1;
}

int64_t cla_add_group_rle(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dict, int32_t nVals,
                          const int32_t* ptr, const uint16_t* data, int64_t dataLen) {
  return add_offset_group(h, GT_RLE, colIdx, gCols, dict, nVals, ptr, data, dataLen);
}
int64_t cla_add_group_ole(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dict, int32_t nVals,
                          const int32_t* ptr, const uint16_t* data, int64_t dataLen) {
  return add_offset_group(h, GT_OLE, colIdx, gCols, dict, nVals, ptr, data, dataLen);
}

int64_t cla_add_group_uncompressed(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* values) {
  GET_MATRIX(h);
  REQUIRE_OPEN();
  int64_t rc = check_cols(m, colIdx, gCols);
  if (rc < 0) return rc;
  if (m->nRows > 0 && !values) return fail(CLA_ERR_BAD_ARG, "dense block missing");
  HostGroup g;
  g.type = GT_UNC;
  g.cols.assign(colIdx, colIdx + gCols);
  if (m->nRows) g.dense.assign(values, values + (size_t)m->nRows * gCols);
  m->hg.push_back(std::move(g));
  return (int64_t)m->hg.size() - 1;
}

// Registration from device memory: the index map / dense block already lives on the GPU (a block that was compressed,
// sliced or generated there). The buffer is read at cla_finalize, which copies it device to device and checks the
// ids with a reduction kernel; it must stay valid and unchanged until cla_finalize has returned.
int64_t cla_add_group_ddc_dev(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dict, int32_t nVals,
                              int32_t mapType, const void* dMap, int64_t mapSize) {
  GET_MATRIX(h);
  REQUIRE_OPEN();
  HostGroup g;
  int64_t rc = add_dict_group(m, g, GT_DDC, colIdx, gCols, dict, nVals);
  if (rc < 0) return rc;
  if (mapSize != m->nRows) return fail(CLA_ERR_SHAPE, "DDC map must have one cell per row");
  if (m->nRows > 0 && nVals == 0) return fail(CLA_ERR_BAD_ARG, "DDC group without dictionary tuples");
  if (mapType != CLA_MAP_BIT && mapType != CLA_MAP_UBYTE && mapType != CLA_MAP_BYTE && mapType != CLA_MAP_CHAR &&
      mapType != CLA_MAP_INT)
    return fail(CLA_ERR_UNSUPPORTED, "device-resident maps: MapToBit, MapToUByte, MapToByte, MapToChar or MapToInt");
  if (mapSize > 0 && !dMap) return fail(CLA_ERR_BAD_ARG, "map array missing");
  cudaPointerAttributes at{};
  if (mapSize > 0 && (cudaPointerGetAttributes(&at, dMap) != cudaSuccess || at.type != cudaMemoryTypeDevice)) {
    cudaGetLastError();
    return fail(CLA_ERR_BAD_ARG, "device-resident map: not a device pointer");
  }
  g.mapType = mapType;
  g.mapSize = mapSize;
  g.devMap = dMap;
  g.devSrcDevice = mapSize > 0 ? at.device : -1;
  m->hg.push_back(std::move(g));
  return (int64_t)m->hg.size() - 1;
}

int64_t cla_add_group_uncompressed_dev(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dValues) {
  GET_MATRIX(h);
  REQUIRE_OPEN();
  int64_t rc = check_cols(m, colIdx, gCols);
  if (rc < 0) return rc;
  if (m->nRows > 0 && !dValues) return fail(CLA_ERR_BAD_ARG, "dense block missing");
  cudaPointerAttributes at{};
  if (m->nRows > 0 && (cudaPointerGetAttributes(&at, dValues) != cudaSuccess || at.type != cudaMemoryTypeDevice)) {
    cudaGetLastError();
    return fail(CLA_ERR_BAD_ARG, "device-resident dense block: not a device pointer");
  }
  HostGroup g;
  g.type = GT_UNC;
  g.cols.assign(colIdx, colIdx + gCols);
  g.devDense = dValues;
  g.devSrcDevice = m->nRows > 0 ? at.device : -1;
  m->hg.push_back(std::move(g));
  return (int64_t)m->hg.size() - 1;
}

int64_t cla_add_group_const(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* tuple) {
  GET_MATRIX(h);
  REQUIRE_OPEN();
  HostGroup g;
  int64_t rc = add_dict_group(m, g, GT_CONST, colIdx, gCols, tuple, 1);
  if (rc < 0) return rc;
  m->hg.push_back(std::move(g));
  return (int64_t)m->hg.size() - 1;
}

int64_t cla_add_group_empty(cla_handle h, const int32_t* colIdx, int32_t gCols) {
  GET_MATRIX(h);
  REQUIRE_OPEN();
  int64_t rc = check_cols(m, colIdx, gCols);
  if (rc < 0) return rc;
  HostGroup g;
  g.type = GT_EMPTY;
  g.cols.assign(colIdx, colIdx + gCols);
  m->hg.push_back(std::move(g));
  return (int64_t)m->hg.size() - 1;
}

int64_t cla_finalize(cla_handle h, int32_t device) {
  GET_MATRIX(h);
  REQUIRE_OPEN();
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(CLA_ERR_CUDA, std::string("no usable CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0"));
  if (device < 0 || device >= count) return fail(CLA_ERR_BAD_ARG, "device ordinal out of range");
  m->device = device;
  int64_t rc = finalize_device(m);
  if (rc < 0) {
    release(m);
    m->device = -1;
    return rc;
  }
  return CLA_OK;
}

}  // extern "C"

// ---- device-buffer products ---------------------------------------------------------------------
static int64_t check_errword(Matrix* m) {
  int32_t herr = 0;
  CLA_CUDA(cudaMemcpy(&herr, m->dErr, sizeof(herr), cudaMemcpyDeviceToHost));
  if (herr) {
    cudaMemset(m->dErr, 0, sizeof(int32_t));
    return fail(CLA_ERR_DEVICE_CHECK, "a kernel self-check tripped (code " + std::to_string(herr) + ")");
  }
  return CLA_OK;
}

// Few right-hand columns (or few left-hand rows) are served by the one-vector kernels, once per vector: each
// pass re-reads the maps, which is cheaper than the general tile kernels up to the limits below.
static int loop_limit(const char* env, int dflt) {
  const char* e = getenv(env);
  return e ? atoi(e) : dflt;
}

__global__ void k_small_transpose(const double* __restrict__ in, int rows, int cols, double* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows * cols) out[(size_t)(i % cols) * rows + i / cols] = in[i];
}

// U holds vCols result vectors of nRows each; out is row-major nRows x vCols.
__global__ void k_vectors_to_rows(const double* __restrict__ U, int64_t nRows, int64_t stride, int vCols,
                                  double* __restrict__ out) {
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < nRows; r += (int64_t)gridDim.x * blockDim.x)
    for (int j = 0; j < vCols; j++) out[r * vCols + j] = U[(int64_t)j * stride + r];
}

static int64_t rmm_by_vectors(Matrix* m, const double* dV, int32_t vCols, double* dOut, cudaStream_t s) {
  const size_t vtBytes = (((size_t)vCols * m->nCols * sizeof(double)) + 255) & ~(size_t)255;
  const size_t rowsPad = ((size_t)m->nRows + 31) & ~(size_t)31;
  int64_t rc = ensure_scratch2(m, vtBytes + rowsPad * vCols * sizeof(double));
  if (rc < 0) return rc;
  double* Vt = (double*)m->scratch2;
  double* U = (double*)((char*)m->scratch2 + vtBytes);
  const int cells = m->nCols * vCols;
  k_small_transpose<<<(cells + 255) / 256, 256, 0, s>>>(dV, m->nCols, vCols, Vt);
  for (int j = 0; j < vCols; j++) {
    double* uj = U + rowsPad * j;
    rc = fast_rmm_vec(m, Vt + (size_t)j * m->nCols, uj, s);
    if (rc < 0) return rc;
    if (rc == 2) rc = launch_rmm(m, Vt + (size_t)j * m->nCols, 1, uj, s, true);
    else if (rc == 0) rc = launch_rmm(m, Vt + (size_t)j * m->nCols, 1, uj, s);
    if (rc < 0) return rc;
  }
  k_vectors_to_rows<<<m->smCount * 8, 256, 0, s>>>(U, m->nRows, (int64_t)rowsPad, vCols, dOut);
  m->stats.kernel_launches += 2;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

static int64_t rmm_dev(Matrix* m, const double* dV, int32_t vRows, int32_t vCols, double* dOut, cudaStream_t s) {
  if (vRows != m->nCols) return fail(CLA_ERR_SHAPE, "rmm: V must have nCols rows");
  if (vCols < 0) return fail(CLA_ERR_SHAPE, "rmm: negative column count");
  m->stats.calls_rmm++;
  if (vCols == 1) {
    int64_t rc = fast_rmm_vec(m, dV, dOut, s);
    if (rc < 0) return rc;
    if (rc == 1) return CLA_OK;
    return launch_rmm(m, dV, 1, dOut, s, rc == 2);
  }
  // A pass of the one-column kernels per column beats the tensor-core kernel (whose time hardly depends on
  // the width up to 64 columns) for a few columns; measured crossover: about 16 columns when every group is
  // a byte-map DDC group (2M x 200: 0.26 ms per column against 4.3 ms), about 7 when SDC / RLE groups take
  // the general pass as well (1M x 500, 451 groups: 0.25 ms per column against 1.9 ms).
  static const int loopEnv = loop_limit("CLA_RMM_LOOP_MAX", -1);  // tuning aid
  const int loopMax = loopEnv >= 0 ? loopEnv : (fast_plan_partial(m) ? 7 : 12);
  if (vCols >= 2 && vCols <= loopMax && fast_plan_ok(m) && m->nRows > 0) return rmm_by_vectors(m, dV, vCols, dOut, s);
  return launch_rmm_dmma(m, dV, vCols, dOut, s);  // FP64 tensor cores
}

static int64_t lmm_dev(Matrix* m, const double* dYt, int32_t yRows, double* dOut, cudaStream_t s) {
  if (yRows < 0) return fail(CLA_ERR_SHAPE, "lmm: negative row count");
  m->stats.calls_lmm++;
  if (yRows == 1) {
    int64_t rc = fast_lmm_vec(m, dYt, dOut, s);
    if (rc < 0) return rc;
    if (rc == 1) return CLA_OK;
    if (rc == 2) return launch_lmm(m, dYt, yRows, dOut, s, true);
  }
  // Several left rows: passes of the column-per-lane kernels over four, two or one row at a time for the groups they
  // cover (measured 0.17 ms per row on 2M x 200 for the one-row kernel against 1.5 ms per row in the general
  // pre-aggregation kernel), the general kernels for the rest. Rows of an odd-length Yt are not 16-byte aligned, so they are copied to a padded pitch first.
  static const int lmmLoopMax = loop_limit("CLA_LMM_LOOP_MAX", 1 << 30);  // tuning aid
  if (yRows >= 2 && yRows <= lmmLoopMax && fast_plan_ok(m) && m->nRows > 0) {
    const double* rows = dYt;
    size_t pitch = (size_t)m->nRows;
    if (m->nRows & 1) {
      pitch = (size_t)m->nRows + 1;
      int64_t rc = ensure_scratch2(m, pitch * yRows * sizeof(double));
      if (rc < 0) return rc;
      CLA_CUDA(cudaMemcpy2DAsync(m->scratch2, pitch * sizeof(double), dYt, (size_t)m->nRows * sizeof(double),
                                 (size_t)m->nRows * sizeof(double), yRows, cudaMemcpyDeviceToDevice, s));
      rows = (const double*)m->scratch2;
    }
    int64_t rc = 0;
    for (int i = 0; i < yRows;) {  // four rows per pass over the maps, then two, then one
      const int q = yRows - i >= 4 ? 4 : (yRows - i >= 2 ? 2 : 1);
      rc = q == 1 ? fast_lmm_vec(m, rows + pitch * i, dOut + (size_t)i * m->nCols, s)
                  : fast_lmm_rows(m, rows + pitch * i, pitch, q, dOut + (size_t)i * m->nCols, s);
      if (rc <= 0) break;
      i += q;
    }
    if (rc < 0) return rc;
    if (rc == 1) return CLA_OK;
    if (rc == 2) return launch_lmm(m, dYt, yRows, dOut, s, true);
  }
  return launch_lmm(m, dYt, yRows, dOut, s);
}

static int64_t mmchain_dev(Matrix* m, const double* dV, const double* dW, int32_t ctype, double* dOut, double* dU,
                           cudaStream_t s) {
  if (ctype != CLA_CHAIN_XtXv && ctype != CLA_CHAIN_XtwXv) return fail(CLA_ERR_UNSUPPORTED, "mmchain: unsupported chain type");
  if (ctype == CLA_CHAIN_XtwXv && !dW) return fail(CLA_ERR_BAD_ARG, "mmchain: XtwXv needs w");
  m->stats.calls_mmchain++;
  if (!dU) {
    int64_t rc = ensure_scratch2(m, sizeof(double) * (size_t)std::max(m->nRows, 1));
    if (rc < 0) return rc;
    dU = (double*)m->scratch2;
  }
  int64_t rc = rmm_dev(m, dV, m->nCols, 1, dU, s);
  if (rc < 0) return rc;
  if (ctype == CLA_CHAIN_XtwXv)
    if ((rc = launch_scale_rows(m, dU, dW, m->nRows, s)) < 0) return rc;
  return lmm_dev(m, dU, 1, dOut, s);
}

// Device-buffer calls return once their work is enqueued. All calls on a handle share its scratch buffers, so
// a call on another stream than the handle's previous call is made to wait for that call on the device.
template <class F>
static int64_t ordered(Matrix* m, cudaStream_t s, F&& run) {
  int64_t rc = order_begin(m, s);
  if (rc < 0) return rc;
  rc = run();
  const int64_t rc2 = order_end(m, s);  // also after a failed launch sequence: part of it may be enqueued
  return rc < 0 ? rc : (rc2 < 0 ? rc2 : rc);
}

extern "C" {

int64_t cla_rmm_dev(cla_handle h, const double* dV, int32_t vRows, int32_t vCols, double* dOut, void* stream) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  CLA_CUDA(cudaSetDevice(m->device));
  cudaStream_t s = (cudaStream_t)stream;
  return ordered(m, s, [&] { return rmm_dev(m, dV, vRows, vCols, dOut, s); });
}
int64_t cla_lmm_dev(cla_handle h, const double* dYt, int32_t yRows, double* dOut, void* stream) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  CLA_CUDA(cudaSetDevice(m->device));
  cudaStream_t s = (cudaStream_t)stream;
  return ordered(m, s, [&] { return lmm_dev(m, dYt, yRows, dOut, s); });
}
int64_t cla_lmm_vec_noalloc_dev(cla_handle h, const double* dY, double* dOut, void* stream) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  CLA_CUDA(cudaSetDevice(m->device));
  if (!dY || !dOut) return fail(CLA_ERR_BAD_ARG, "no-allocation product: null buffer");
  cudaStream_t s = (cudaStream_t)stream;
  return ordered(m, s, [&] { return fast_lmm_vec_noalloc(m, dY, dOut, s); });
}
int64_t cla_tsmm_dev(cla_handle h, double* dOut, void* stream) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  CLA_CUDA(cudaSetDevice(m->device));
  m->stats.calls_tsmm++;
  cudaStream_t s = (cudaStream_t)stream;
  return ordered(m, s, [&] { return launch_tsmm(m, dOut, s); });
}
int64_t cla_decompress_dev(cla_handle h, double* dOut, void* stream) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  CLA_CUDA(cudaSetDevice(m->device));
  m->stats.calls_decompress++;
  cudaStream_t s = (cudaStream_t)stream;
  return ordered(m, s, [&] { return launch_decompress(m, dOut, s); });
}
int64_t cla_mmchain_dev(cla_handle h, const double* dV, const double* dW, int32_t ctype, double* dOut, double* dU,
                        void* stream) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  CLA_CUDA(cudaSetDevice(m->device));
  cudaStream_t s = (cudaStream_t)stream;
  return ordered(m, s, [&] { return mmchain_dev(m, dV, dW, ctype, dOut, dU, s); });
}

}  // extern "C"

// ---- host-buffer products -------------------------------------------------------------------------
// Staging layout in m->io: [inputs ... | output | nnz counter]
template <class F>
static int64_t host_call(Matrix* m, const double* in1, size_t n1, const double* in2, size_t n2, double* out, size_t nOut,
                         F&& run, bool deferIn1 = false) {
  CLA_CUDA(cudaSetDevice(m->device));
  auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
  const size_t o1 = 0, o2 = al(n1 * 8), oOut = o2 + al(n2 * 8), oCnt = oOut + al(nOut * 8);
  int64_t rc = ensure_io(m, oCnt + 256);
  if (rc < 0) return rc;
  char* base = (char*)m->io;
  double* d1 = (double*)(base + o1);
  double* d2 = (double*)(base + o2);
  double* dOut = (double*)(base + oOut);
  unsigned long long* dCnt = (unsigned long long*)(base + oCnt);
  cudaStream_t s = m->stream;
  if ((rc = order_begin(m, s)) < 0) return rc;
  // large operands in pageable memory go through the handle's pinned ring (cla_hostcopy.cu)
  auto upload = [&](double* d, const double* h, size_t n) -> int64_t {
    if (host_copy_staged(m, h, n * 8)) return host_to_device_staged(m, d, h, n * 8, s, nullptr);
    CLA_CUDA(cudaMemcpyAsync(d, h, n * 8, cudaMemcpyHostToDevice, s));
    return CLA_OK;
  };
  if (n1 && !deferIn1 && (rc = upload(d1, in1, n1)) < 0) return rc;  // deferred: run() uploads it
  if (n2 && (rc = upload(d2, in2, n2)) < 0) return rc;
  CLA_CUDA(cudaEventRecord(m->ev0, s));
  if ((rc = run(d1, n2 ? d2 : nullptr, dOut, s)) < 0) return rc;
  CLA_CUDA(cudaEventRecord(m->ev1, s));
  if ((rc = launch_count_nnz(m, dOut, (int64_t)nOut, dCnt, s)) < 0) return rc;
  if (nOut) {
    if (host_copy_staged(m, out, nOut * 8)) {
      if ((rc = device_to_host_staged(m, out, dOut, nOut * 8, s)) < 0) return rc;
    } else
      CLA_CUDA(cudaMemcpyAsync(out, dOut, nOut * 8, cudaMemcpyDeviceToHost, s));
  }
  unsigned long long nnz = 0;
  CLA_CUDA(cudaMemcpyAsync(&nnz, dCnt, sizeof(nnz), cudaMemcpyDeviceToHost, s));
  CLA_CUDA(cudaStreamSynchronize(s));
  m->lastValid = false;  // nothing of this handle is in flight any more
  float ms = 0;
  if (cudaEventElapsedTime(&ms, m->ev0, m->ev1) == cudaSuccess) m->stats.last_kernel_ms = ms;
  if ((rc = check_errword(m)) < 0) return rc;
  return (int64_t)nnz;
}

// Two handles for one product: both are looked up, locked in address order (so two concurrent calls with the
// operands swapped cannot deadlock) and checked to be finalized on the same device over the same rows.
struct PairLock {
  std::shared_ptr<Matrix> l, r;
  std::unique_lock<std::mutex> k1, k2;
};
static int64_t lock_pair(cla_handle hl, cla_handle hr, PairLock& p) {
  p.l = lookup(hl);
  p.r = lookup(hr);
  if (!p.l || !p.r) return fail(CLA_ERR_BAD_HANDLE, "unknown or destroyed handle");
  Matrix *a = p.l.get(), *b = p.r.get();
  if (a == b)
    p.k1 = std::unique_lock<std::mutex>(a->mu);
  else {
    Matrix *first = a < b ? a : b, *second = a < b ? b : a;
    p.k1 = std::unique_lock<std::mutex>(first->mu);
    p.k2 = std::unique_lock<std::mutex>(second->mu);
  }
  if (!a->finalized || !b->finalized) return fail(CLA_ERR_STATE, "cla_finalize has not been called on both handles");
  if (a->device != b->device) return fail(CLA_ERR_BAD_ARG, "tmm: both blocks must be on the same device");
  if (a->nRows != b->nRows) return fail(CLA_ERR_SHAPE, "tmm: the blocks must have the same number of rows");
  return CLA_OK;
}
static int64_t tmm_dev(Matrix* l, Matrix* r, double* dOut, cudaStream_t s) {
  l->stats.calls_tsmm++;
  if (l == r) return launch_tsmm(l, dOut, s);  // one block on both sides: the symmetric kernel
  return launch_tmm(l, r, dOut, s);
}

extern "C" {

int64_t cla_tmm(cla_handle left, cla_handle right, double* out) {
  PairLock p;
  int64_t rc = lock_pair(left, right, p);
  if (rc < 0) return rc;
  Matrix *l = p.l.get(), *r = p.r.get();
  if (!out && (size_t)l->nCols * r->nCols) return fail(CLA_ERR_BAD_ARG, "tmm: null buffer");
  if (r != l && l->stream) {
    CLA_CUDA(cudaSetDevice(l->device));
    if ((rc = order_begin(r, l->stream)) < 0) return rc;
  }
  rc = host_call(l, nullptr, 0, nullptr, 0, out, (size_t)l->nCols * r->nCols,
                 [&](double*, double*, double* dOut, cudaStream_t s) { return tmm_dev(l, r, dOut, s); });
  if (r != l && rc >= 0) r->lastValid = false;  // host_call synchronised the stream both blocks' kernels ran on
  return rc;
}

int64_t cla_tmm_dev(cla_handle left, cla_handle right, double* dOut, void* stream) {
  PairLock p;
  int64_t rc = lock_pair(left, right, p);
  if (rc < 0) return rc;
  CLA_CUDA(cudaSetDevice(p.l->device));
  cudaStream_t s = (cudaStream_t)stream;
  Matrix *l = p.l.get(), *r = p.r.get();
  if ((rc = order_begin(l, s)) < 0) return rc;
  if (r != l && (rc = order_begin(r, s)) < 0) return rc;
  rc = tmm_dev(l, r, dOut, s);
  const int64_t e1 = order_end(l, s), e2 = r != l ? order_end(r, s) : CLA_OK;
  return rc < 0 ? rc : (e1 < 0 ? e1 : (e2 < 0 ? e2 : rc));
}

// X %*% V as an overlapping compressed block (see make_overlapping)
static cla_handle rmm_overlapping(cla_handle h, const double* V, bool vOnDevice, int32_t vRows, int32_t vCols, cudaStream_t userStream) {
  std::shared_ptr<Matrix> mp = lookup(h);
  if (!mp) return fail(CLA_ERR_BAD_HANDLE, "unknown or destroyed handle");
  Matrix* m = mp.get();
  std::lock_guard<std::mutex> lk(m->mu);
  if (!m->finalized) return fail(CLA_ERR_STATE, "cla_finalize has not been called on this handle");
  if (vRows != m->nCols || vCols < 0) return fail(CLA_ERR_SHAPE, "rmm: V must be [nCols x vCols]");
  if (!V && (size_t)vRows * vCols) return fail(CLA_ERR_BAD_ARG, "rmm: null buffer");
  CLA_CUDA(cudaSetDevice(m->device));
  cudaStream_t s = vOnDevice ? userStream : m->stream;
  int64_t rc;
  if ((rc = order_begin(m, s)) < 0) return rc;
  const double* dV = V;
  if (!vOnDevice) {
    const size_t bytes = (size_t)vRows * vCols * sizeof(double);
    if ((rc = ensure_io(m, bytes + 256)) < 0) return rc;
    if (bytes) CLA_CUDA(cudaMemcpyAsync(m->io, V, bytes, cudaMemcpyHostToDevice, s));
    dV = (const double*)m->io;
  }
  auto child = std::make_shared<Matrix>();
  m->stats.calls_rmm++;
  rc = make_overlapping(m, child.get(), dV, vCols, s);  // synchronises s
  m->lastValid = false;
  if (rc < 0) {
    release(child.get());
    return rc;
  }
  child->parent = mp;
  m->children++;
  return table_insert(child);
}

cla_handle cla_rmm_overlapping(cla_handle h, const double* V, int32_t vRows, int32_t vCols) {
  return rmm_overlapping(h, V, false, vRows, vCols, nullptr);
}
cla_handle cla_rmm_overlapping_dev(cla_handle h, const double* dV, int32_t vRows, int32_t vCols, void* stream) {
  return rmm_overlapping(h, dV, true, vRows, vCols, (cudaStream_t)stream);
}

int64_t cla_rmm(cla_handle h, const double* V, int32_t vRows, int32_t vCols, double* out) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  if (vRows != m->nCols || vCols < 0) return fail(CLA_ERR_SHAPE, "rmm: V must be [nCols x vCols]");
  if ((!V && (size_t)vRows * vCols) || (!out && (size_t)m->nRows * vCols)) return fail(CLA_ERR_BAD_ARG, "rmm: null buffer");
  return host_call(m, V, (size_t)vRows * vCols, nullptr, 0, out, (size_t)m->nRows * vCols,
                   [&](double* dV, double*, double* dOut, cudaStream_t s) { return rmm_dev(m, dV, vRows, vCols, dOut, s); });
}

int64_t cla_lmm(cla_handle h, const double* Yt, int32_t yRows, double* out) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  if (yRows < 0) return fail(CLA_ERR_SHAPE, "lmm: negative row count");
  if ((!Yt && (size_t)yRows * m->nRows) || (!out && (size_t)yRows * m->nCols)) return fail(CLA_ERR_BAD_ARG, "lmm: null buffer");
  if (yRows == 1)  // one left row: upload it in slices that overlap with the product where the kernel allows
    return host_call(
        m, Yt, (size_t)m->nRows, nullptr, 0, out, (size_t)m->nCols,
        [&](double* dY, double*, double* dOut, cudaStream_t s) -> int64_t {
          m->stats.calls_lmm++;
          int64_t rc = fast_lmm_vec_host(m, Yt, dY, dOut, s);
          if (rc != 0) return rc < 0 ? rc : CLA_OK;
          m->stats.calls_lmm--;
          if (m->nRows) CLA_CUDA(cudaMemcpyAsync(dY, Yt, (size_t)m->nRows * 8, cudaMemcpyHostToDevice, s));
          return lmm_dev(m, dY, 1, dOut, s);
        },
        true);
  return host_call(m, Yt, (size_t)yRows * m->nRows, nullptr, 0, out, (size_t)yRows * m->nCols,
                   [&](double* dY, double*, double* dOut, cudaStream_t s) { return lmm_dev(m, dY, yRows, dOut, s); });
}

int64_t cla_tsmm(cla_handle h, double* out) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  if (!out && m->nCols) return fail(CLA_ERR_BAD_ARG, "tsmm: null buffer");
  m->stats.calls_tsmm++;
  return host_call(m, nullptr, 0, nullptr, 0, out, (size_t)m->nCols * m->nCols,
                   [&](double*, double*, double* dOut, cudaStream_t s) { return launch_tsmm(m, dOut, s); });
}

int64_t cla_mmchain(cla_handle h, const double* v, const double* w, int32_t ctype, double* out) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  if ((!v || !out) && m->nCols) return fail(CLA_ERR_BAD_ARG, "mmchain: null buffer");
  if (ctype == CLA_CHAIN_XtwXv && !w && m->nRows) return fail(CLA_ERR_BAD_ARG, "mmchain: XtwXv needs w");
  const size_t nW = ctype == CLA_CHAIN_XtwXv ? (size_t)m->nRows : 0;
  return host_call(m, v, (size_t)m->nCols, w, nW, out, (size_t)m->nCols,
                   [&](double* dV, double* dW, double* dOut, cudaStream_t s) {
                     return mmchain_dev(m, dV, dW, ctype, dOut, nullptr, s);
                   });
}

// Column sums are t(1) %*% X and row sums X %*% 1, so both run on the product kernels.
int64_t cla_unary_agg(cla_handle h, int32_t op, double* out) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  if (op < CLA_AGG_COL_SUMS || op > CLA_AGG_MAX) return fail(CLA_ERR_BAD_ARG, "unary aggregate: unknown operation");
  if (!out) return fail(CLA_ERR_BAD_ARG, "unary aggregate: null buffer");
  if (op == CLA_AGG_ROW_MINS || op == CLA_AGG_ROW_MAXS)
    return host_call(m, nullptr, 0, nullptr, 0, out, (size_t)m->nRows, [&](double*, double*, double* dOut, cudaStream_t s) {
      return row_minmax(m, op == CLA_AGG_ROW_MAXS, dOut, s);
    });
  if (op >= CLA_AGG_COL_MINS) {
    CLA_CUDA(cudaSetDevice(m->device));
    std::vector<double> lo, hi;
    int64_t rc = col_minmax(m, lo, hi, m->stream);
    if (rc < 0) return rc;
    if ((rc = check_errword(m)) < 0) return rc;
    const bool wantMax = (op == CLA_AGG_COL_MAXS || op == CLA_AGG_MAX);
    const std::vector<double>& v = wantMax ? hi : lo;
    int64_t nnz = 0;
    if (op == CLA_AGG_MIN || op == CLA_AGG_MAX) {
      // an empty block aggregates to 0 like an empty MatrixBlock (runtime/matrix/data/MatrixBlock.java min / max)
      double r = (m->nRows == 0 || m->nCols == 0) ? 0.0 : (wantMax ? -INFINITY : INFINITY);
      if (m->nRows > 0)
        for (double x : v) r = wantMax ? std::fmax(r, x) : std::fmin(r, x);
      out[0] = r;
      return r != 0.0 ? 1 : 0;
    }
    for (int c = 0; c < m->nCols; c++) {
      out[c] = m->nRows == 0 ? 0.0 : v[c];
      nnz += out[c] != 0.0;
    }
    return nnz;
  }
  if (op == CLA_AGG_ROW_SUMS) {
    std::vector<double> ones((size_t)m->nCols, 1.0);
    return host_call(m, ones.data(), ones.size(), nullptr, 0, out, (size_t)m->nRows,
                     [&](double* dV, double*, double* dOut, cudaStream_t s) { return rmm_dev(m, dV, m->nCols, 1, dOut, s); });
  }
  std::vector<double> ones((size_t)m->nRows, 1.0), cs((size_t)m->nCols, 0.0);
  int64_t rc = host_call(m, ones.data(), ones.size(), nullptr, 0, op == CLA_AGG_SUM ? cs.data() : out, (size_t)m->nCols,
                         [&](double* dY, double*, double* dOut, cudaStream_t s) { return lmm_dev(m, dY, 1, dOut, s); });
  if (rc < 0 || op == CLA_AGG_COL_SUMS) return rc;
  double total = 0;
  for (double x : cs) total += x;
  out[0] = total;
  return total != 0.0 ? 1 : 0;
}

int64_t cla_decompress(cla_handle h, double* out) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  if (!out && (size_t)m->nRows * m->nCols) return fail(CLA_ERR_BAD_ARG, "decompress: null buffer");
  m->stats.calls_decompress++;
  return host_call(m, nullptr, 0, nullptr, 0, out, (size_t)m->nRows * m->nCols,
                   [&](double*, double*, double* dOut, cudaStream_t s) { return launch_decompress(m, dOut, s); });
}

// ---- decoded index structures -----------------------------------------------------------------------
int64_t cla_group_decode(cla_handle h, int32_t g, int32_t* ids) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  if (g < 0 || g >= (int)m->regToDev.size()) return fail(CLA_ERR_BAD_ARG, "group index out of range");
  if (!ids && m->nRows) return fail(CLA_ERR_BAD_ARG, "null buffer");
  if (m->nRows == 0) return CLA_OK;
  CLA_CUDA(cudaSetDevice(m->device));
  const int dg = m->regToDev[g];
  if (dg < 0) {  // const: tuple 0 everywhere; empty: no tuple
    const int v = m->hg[g].type == GT_CONST ? 0 : -1;
    for (int r = 0; r < m->nRows; r++) ids[r] = v;
    return CLA_OK;
  }
  int64_t rc = ensure_io(m, sizeof(int32_t) * (size_t)m->nRows);
  if (rc < 0) return rc;
  if ((rc = launch_group_decode(m, dg, (int32_t*)m->io, m->stream)) < 0) return rc;
  CLA_CUDA(cudaMemcpyAsync(ids, m->io, sizeof(int32_t) * (size_t)m->nRows, cudaMemcpyDeviceToHost, m->stream));
  CLA_CUDA(cudaStreamSynchronize(m->stream));
  return CLA_OK;
}

int64_t cla_group_counts(cla_handle h, int32_t g, int64_t* counts) {
  GET_MATRIX(h);
  REQUIRE_FINAL();
  if (g < 0 || g >= (int)m->regToDev.size()) return fail(CLA_ERR_BAD_ARG, "group index out of range");
  if (!counts) return fail(CLA_ERR_BAD_ARG, "null buffer");
  CLA_CUDA(cudaSetDevice(m->device));
  const int dg = m->regToDev[g];
  if (dg < 0) {
    if (m->hg[g].type == GT_CONST) counts[0] = m->nRows;
    return CLA_OK;
  }
  const int nv = m->hg[g].nVals;
  if (m->groups[dg].type == GT_UNC) return fail(CLA_ERR_UNSUPPORTED, "counts: uncompressed group has no dictionary");
  int64_t rc = ensure_io(m, sizeof(unsigned long long) * (size_t)std::max(nv + 1, 1));
  if (rc < 0) return rc;
  if ((rc = launch_group_counts(m, dg, (unsigned long long*)m->io, m->stream)) < 0) return rc;
  CLA_CUDA(cudaMemcpyAsync(counts, m->io, sizeof(int64_t) * (size_t)nv, cudaMemcpyDeviceToHost, m->stream));
  CLA_CUDA(cudaStreamSynchronize(m->stream));
  return CLA_OK;
}

}  // extern "C"
