// t(X) %*% X on a compressed matrix (CLALibTSMM.leftMultByTransposeSelf, lib/CLALibTSMM.java:59-94).
//
// The reference multiplies dictionaries when there are few groups and otherwise decompresses the
// whole matrix and runs a dense self product (:73-77). Here the second strategy is used for all
// inputs, but blocked so the dense form never exists in full: a chunk of rows small enough to stay
// resident in L2 is decompressed into scratch, an FP64 tensor-core (DMMA m8n8k4) SYRK adds
// chunk^T * chunk into the upper 64 x 64 blocks of the result, and the next chunk reuses the scratch.
// Constant columns are part of the decompressed chunk, so no correction layer is needed.
#include "cla_common.cuh"
#include <algorithm>

namespace cla {

constexpr int TS_BLK = 64;      // C block edge
constexpr int TS_KT = 16;       // rows per shared-memory stage
constexpr int TS_LD = 68;       // padded row stride (doubles): k * 68 mod 16 = {0,4,8,12} keeps fragment loads conflict free
constexpr int TS_THREADS = 256;

__device__ __forceinline__ void dmma884(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c0), "+d"(c1)
               : "d"(a), "d"(b));
}

// grid: (upper block pairs, k splits). X: [rows x nCols] row-major chunk. C += X^T X (upper blocks only).
__global__ void __launch_bounds__(TS_THREADS)
k_syrk_dmma(const double* __restrict__ X, int rows, int nCols, int nBlk, double* __restrict__ C, int rowsPerSplit) {
  __shared__ double sI[TS_KT * TS_LD];
  __shared__ double sJ[TS_KT * TS_LD];
  // decode the linear pair index into (bi <= bj)
  int p = blockIdx.x, bi = 0;
  while (p >= nBlk - bi) {
    p -= nBlk - bi;
    bi++;
  }
  const int bj = bi + p;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rBeg = blockIdx.y * rowsPerSplit, rEnd = min(rows, rBeg + rowsPerSplit);
  double c[8][2];
#pragma unroll
  for (int t = 0; t < 8; t++) c[t][0] = c[t][1] = 0.0;
  const int am = lane >> 2, ak = lane & 3;
  for (int r = rBeg; r < rEnd; r += TS_KT) {
    // stage KT rows of column blocks bi and bj (zero padded)
    for (int e = tid; e < TS_KT * TS_BLK; e += TS_THREADS) {
      const int kk = e / TS_BLK, cc = e - kk * TS_BLK;
      const int row = r + kk;
      const int ci = bi * TS_BLK + cc, cj = bj * TS_BLK + cc;
      sI[kk * TS_LD + cc] = (row < rEnd && ci < nCols) ? X[(size_t)row * nCols + ci] : 0.0;
      sJ[kk * TS_LD + cc] = (row < rEnd && cj < nCols) ? X[(size_t)row * nCols + cj] : 0.0;
    }
    __syncthreads();
#pragma unroll
    for (int k0 = 0; k0 < TS_KT; k0 += 4) {
      const double a = sI[(k0 + ak) * TS_LD + warp * 8 + am];  // A[m][k] = X[k][bi*64 + warp*8 + m]
#pragma unroll
      for (int t = 0; t < 8; t++) {
        const double b = sJ[(k0 + ak) * TS_LD + t * 8 + am];   // B[k][n] = X[k][bj*64 + t*8 + n]
        dmma884(c[t][0], c[t][1], a, b);
      }
    }
    __syncthreads();
  }
  // C fragment: row = lane >> 2, cols = (lane & 3) * 2 + {0, 1}
  const int gi = bi * TS_BLK + warp * 8 + (lane >> 2);
#pragma unroll
  for (int t = 0; t < 8; t++) {
#pragma unroll
    for (int u = 0; u < 2; u++) {
      const int gj = bj * TS_BLK + t * 8 + (lane & 3) * 2 + u;
      if (gi < nCols && gj < nCols && gi <= gj && c[t][u] != 0.0) atomicAdd(&C[(size_t)gi * nCols + gj], c[t][u]);
    }
  }
}

// LibMatrixMult.copyUpperToLowerTriangle (runtime/matrix/data/LibMatrixMult.java:4769-4799)
__global__ void k_mirror(double* __restrict__ C, int n) {
  const int64_t total = (int64_t)n * n;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(e / n), j = (int)(e - (int64_t)i * n);
    if (j < i) C[e] = C[(size_t)j * n + i];
  }
}

int64_t launch_tsmm(Matrix* m, double* dOut, cudaStream_t s) {
  const int n = m->nCols;
  if (n == 0) return CLA_OK;
  CLA_CUDA(cudaMemsetAsync(dOut, 0, sizeof(double) * (size_t)n * n, s));
  if (m->nRows == 0) return CLA_OK;
  // chunk of rows whose dense form stays well inside L2 (48 MB)
  int64_t chunk = (48ll << 20) / ((int64_t)n * 8);
  chunk = std::max<int64_t>(SKIP_ROWS, (chunk / SKIP_ROWS) * SKIP_ROWS);
  chunk = std::min<int64_t>(chunk, ((int64_t)m->nRows + SKIP_ROWS - 1) / SKIP_ROWS * SKIP_ROWS);
  int64_t rc;
  if ((rc = ensure_scratch2(m, (size_t)chunk * n * sizeof(double))) < 0) return rc;
  double* X = (double*)m->scratch2;
  const int nBlk = (n + TS_BLK - 1) / TS_BLK;
  const int nPairs = nBlk * (nBlk + 1) / 2;
  for (int64_t r0 = 0; r0 < m->nRows; r0 += chunk) {
    const int r1 = (int)std::min<int64_t>(m->nRows, r0 + chunk);
    if ((rc = launch_decompress_range(m, (int)r0, r1, X, s)) < 0) return rc;
    const int rows = r1 - (int)r0;
    int splits = std::max(1, std::min((rows + TS_KT * 8 - 1) / (TS_KT * 8), (4 * m->smCount + nPairs - 1) / nPairs));
    int rowsPerSplit = ((rows + splits - 1) / splits + TS_KT - 1) / TS_KT * TS_KT;
    splits = (rows + rowsPerSplit - 1) / rowsPerSplit;
    dim3 grid(nPairs, splits);
    k_syrk_dmma<<<grid, TS_THREADS, 0, s>>>(X, rows, n, nBlk, dOut, rowsPerSplit);
    m->stats.kernel_launches++;
  }
  k_mirror<<<std::max(1, std::min(1024, (int)(((int64_t)n * n + 255) / 256))), 256, 0, s>>>(dOut, n);
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

}  // namespace cla
