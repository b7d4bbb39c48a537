// min / max aggregates of a compressed block: the uamin / uamax / uacmin / uacmax / uarmin / uarmax cases of
// lib/CLALibCompAgg.java.
//
// Column-wise and full aggregates of a non-overlapping block follow the reference's dictionary-based definition
// (colgroup/AColGroupCompressed.java:190-205 -> computeMxx / computeColMxx of each class): the extremum over the
// group's dictionary entries -- every entry counts, whether a row uses it or not -- together with the default tuple
// (ColGroupSDC.java:174-186), with 0 for the classes whose unlisted rows are zero (ColGroupSDCZeros.java:801-812,
// ColGroupSDCSingleZeros.java:595-606) and, for RLE / OLE, with 0 when their runs leave rows uncovered
// (ColGroupRLE.java:723-735). Those per-column pairs are computed on the host when the group is uploaded
// (minmax_of_group); only uncompressed groups need a pass over data (k_dense_col_minmax).
// Row-wise aggregates, and every aggregate of an overlapping block (where the reference decompresses as well,
// lib/CLALibCompAgg.java), run over L2-sized decompressed row chunks.
#include "cla_common.cuh"
#include <algorithm>
#include <cfloat>
#include <cmath>

namespace cla {

// Per-column extrema of one registered group under the dictionary-based definition; called before the default
// tuple is folded into the dictionary.
void minmax_of_group(const HostGroup& hg, int nRows, std::vector<double>& colMin, std::vector<double>& colMax) {
  const int gc = (int)hg.cols.size();
  auto add = [&](int j, double v) {
    colMin[hg.cols[j]] = std::fmin(colMin[hg.cols[j]], v);
    colMax[hg.cols[j]] = std::fmax(colMax[hg.cols[j]], v);
  };
  if (hg.type == GT_UNC) return;  // from the data, on the device
  if (hg.type == GT_EMPTY) {
    for (int j = 0; j < gc; j++) add(j, 0.0);
    return;
  }
  const int nv = hg.type == GT_CONST ? 1 : hg.nVals;
  for (int k = 0; k < nv; k++)
    for (int j = 0; j < gc; j++) add(j, hg.dict[(size_t)k * gc + j]);
  bool zeros = false;
  if (hg.type == GT_SDC) {
    if (hg.def.empty()) zeros = true;
    else
      for (int j = 0; j < gc; j++) add(j, hg.def[j]);
  } else if (hg.type == GT_RLE) {
    int64_t covered = 0;
    for (size_t p = 1; p < hg.data.size(); p += 2) covered += hg.data[p];
    zeros = covered < nRows;
  } else if (hg.type == GT_OLE) {
    int64_t covered = 0;
    for (int k = 0; k < hg.nVals; k++)
      for (int p = hg.ptr[k]; p < hg.ptr[k + 1]; p += hg.data[p] + 1) covered += hg.data[p];
    zeros = covered < nRows;
  }
  if (zeros)
    for (int j = 0; j < gc; j++) add(j, 0.0);
}

// X: [rows x n] row-major. grid (column tiles of 128, row splits); partial extrema per split.
__global__ void k_dense_col_minmax(const double* __restrict__ X, int64_t rows, int n, int64_t rowsPerSplit,
                                   double* __restrict__ pMin, double* __restrict__ pMax) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n) return;
  const int64_t r0 = blockIdx.y * rowsPerSplit, r1 = min(rows, r0 + rowsPerSplit);
  double lo = INFINITY, hi = -INFINITY;
  for (int64_t r = r0; r < r1; r++) {
    const double v = X[r * n + c];
    lo = fmin(lo, v);
    hi = fmax(hi, v);
  }
  pMin[(size_t)blockIdx.y * n + c] = lo;
  pMax[(size_t)blockIdx.y * n + c] = hi;
}

// a warp per row
__global__ void k_dense_row_minmax(const double* __restrict__ X, int64_t rows, int n, double* __restrict__ out, int wantMax) {
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  double v = wantMax ? -INFINITY : INFINITY;
  for (int c = lane; c < n; c += 32) v = wantMax ? fmax(v, X[r * n + c]) : fmin(v, X[r * n + c]);
  for (int d = 16; d; d >>= 1) {
    const double o = __shfl_xor_sync(0xffffffffu, v, d);
    v = wantMax ? fmax(v, o) : fmin(v, o);
  }
  if (lane == 0) out[r] = v;
}

static int64_t dense_col_minmax(Matrix* m, const double* X, int64_t rows, int n, std::vector<double>& lo,
                                std::vector<double>& hi, cudaStream_t s) {
  if (rows <= 0 || n <= 0) return CLA_OK;
  const int splits = (int)std::max<int64_t>(1, std::min<int64_t>(4 * m->smCount, rows / 64));
  const int64_t rps = (rows + splits - 1) / splits;
  int64_t rc = ensure_small(m, (size_t)2 * splits * n * sizeof(double) + 256);
  if (rc < 0) return rc;
  double* pMin = (double*)m->small_;
  double* pMax = pMin + (size_t)splits * n;
  dim3 grid((n + 127) / 128, splits);
  k_dense_col_minmax<<<grid, 128, 0, s>>>(X, rows, n, rps, pMin, pMax);
  m->stats.kernel_launches++;
  std::vector<double> h((size_t)2 * splits * n);
  CLA_CUDA(cudaMemcpyAsync(h.data(), pMin, h.size() * sizeof(double), cudaMemcpyDeviceToHost, s));
  CLA_CUDA(cudaStreamSynchronize(s));
  for (int sp = 0; sp < splits; sp++)
    for (int c = 0; c < n; c++) {
      lo[c] = std::fmin(lo[c], h[(size_t)sp * n + c]);
      hi[c] = std::fmax(hi[c], h[(size_t)(splits + sp) * n + c]);
    }
  return CLA_OK;
}

// Column extrema of the whole block into lo / hi (host vectors of nCols).
int64_t col_minmax(Matrix* m, std::vector<double>& lo, std::vector<double>& hi, cudaStream_t s) {
  const int n = m->nCols;
  lo.assign(n, INFINITY);
  hi.assign(n, -INFINITY);
  if (m->nRows == 0) return CLA_OK;
  int64_t rc;
  if (!m->overlapping && !m->multiCover) {
    lo = m->colMin;
    hi = m->colMax;
    for (auto& g : m->groups)
      if (g.type == GT_UNC) {
        std::vector<double> glo(g.gCols, INFINITY), ghi(g.gCols, -INFINITY);
        if ((rc = dense_col_minmax(m, g.dense, m->nRows, g.gCols, glo, ghi, s)) < 0) return rc;
        std::vector<int32_t> cols(g.gCols);
        CLA_CUDA(cudaMemcpy(cols.data(), g.cols, sizeof(int32_t) * g.gCols, cudaMemcpyDeviceToHost));
        for (int j = 0; j < g.gCols; j++) {
          lo[cols[j]] = std::fmin(lo[cols[j]], glo[j]);
          hi[cols[j]] = std::fmax(hi[cols[j]], ghi[j]);
        }
      }
    for (int c = 0; c < n; c++)
      if (lo[c] > hi[c]) lo[c] = hi[c] = 0.0;  // a column no group holds
    return CLA_OK;
  }
  // overlapping groups (or a frame-of-reference group registered as dictionary group + constant): the extremum
  // of a sum is not the sum of extrema; go through the decompressed rows
  int64_t chunk = std::max<int64_t>(SKIP_ROWS, ((48ll << 20) / ((int64_t)n * 8)) / SKIP_ROWS * SKIP_ROWS);
  chunk = std::min<int64_t>(chunk, ((int64_t)m->nRows + SKIP_ROWS - 1) / SKIP_ROWS * SKIP_ROWS);
  if ((rc = ensure_scratch2(m, (size_t)chunk * n * sizeof(double))) < 0) return rc;
  double* X = (double*)m->scratch2;
  for (int64_t r0 = 0; r0 < m->nRows; r0 += chunk) {
    const int r1 = (int)std::min<int64_t>(m->nRows, r0 + chunk);
    if ((rc = launch_decompress_range(m, (int)r0, r1, X, s)) < 0) return rc;
    if ((rc = dense_col_minmax(m, X, r1 - r0, n, lo, hi, s)) < 0) return rc;
  }
  return CLA_OK;
}

// Row extrema into dOut [nRows] (device).
int64_t row_minmax(Matrix* m, int wantMax, double* dOut, cudaStream_t s) {
  const int n = m->nCols;
  if (m->nRows == 0) return CLA_OK;
  if (n == 0) {
    CLA_CUDA(cudaMemsetAsync(dOut, 0, sizeof(double) * (size_t)m->nRows, s));
    return CLA_OK;
  }
  int64_t rc;
  int64_t chunk = std::max<int64_t>(SKIP_ROWS, ((48ll << 20) / ((int64_t)n * 8)) / SKIP_ROWS * SKIP_ROWS);
  chunk = std::min<int64_t>(chunk, ((int64_t)m->nRows + SKIP_ROWS - 1) / SKIP_ROWS * SKIP_ROWS);
  if ((rc = ensure_scratch2(m, (size_t)chunk * n * sizeof(double))) < 0) return rc;
  double* X = (double*)m->scratch2;
  for (int64_t r0 = 0; r0 < m->nRows; r0 += chunk) {
    const int r1 = (int)std::min<int64_t>(m->nRows, r0 + chunk);
    if ((rc = launch_decompress_range(m, (int)r0, r1, X, s)) < 0) return rc;
    const int64_t rows = r1 - r0;
    k_dense_row_minmax<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(X, rows, n, dOut + r0, wantMax);
    m->stats.kernel_launches++;
  }
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

}  // namespace cla
