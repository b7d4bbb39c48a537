// X %*% V for wide V (8 or more columns) on any mix of groups, on the FP64 tensor cores.
//
// With many right-hand columns the per-row gather-add of the general tile kernel is bound by FP64 adds and
// L1 traffic, not by HBM. Here a CTA owns 128 rows x 64 output columns and
//   1. treats every column of the dense-map (DDC, transcoded OLE) and uncompressed groups as one column of a
//      dense operand: 32 such columns at a time are decoded into shared memory (transposed, so the stores are
//      conflict free) next to the matching 32 rows of V, and multiplied with DMMA m8n8k4 -- this replaces
//      dictionary pre-aggregation + decompress-and-sum (lib/CLALibRightMultBy.java:208-258) for those groups;
//   2. adds the SDC groups from their pre-aggregated tables P_g = D_g * V[cols_g, :] (as the reference does,
//      colgroup/ADictBasedColGroup.java:246-275), one listed row at a time;
//   3. adds the RLE groups from their tables with run-boundary deltas: a run that covers the whole tile goes into
//      one per-tile base vector, only runs that start or end inside the tile touch individual rows;
//   4. adds constV * V and stores.
#include "cla_common.cuh"
#include <algorithm>

namespace cla {

constexpr int GM_TR = 128;     // rows per CTA
constexpr int GM_TN = 64;      // output columns per CTA
constexpr int GM_KC = 32;      // dense columns per stage
constexpr int GM_LDA = 132;    // A^T row stride (doubles), = 4 mod 16: conflict-free fragment loads
constexpr int GM_LDB = 68;     // V tile row stride, = 4 mod 16
constexpr int GM_LDC = 66;     // C tile row stride
constexpr int GM_THREADS = 256;

__device__ __forceinline__ void dmma884(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c0), "+d"(c1)
               : "d"(a), "d"(b));
}

struct DenseCol {
  int32_t group;  // device group index
  int32_t j;      // column inside the group
  int32_t col;    // matrix column (row of V)
  int32_t pad;
};

__global__ void __launch_bounds__(GM_THREADS, 2)
k_rmm_dmma(const DevGroup* __restrict__ groups, int nGroups, const DenseCol* __restrict__ dcols, int nDense, int nRows,
           const double* __restrict__ V, int vCols, const double* __restrict__ P, const double* __restrict__ constRow,
           double* __restrict__ out, int hasSparse) {
  extern __shared__ __align__(16) double sm[];
  double* At = sm;                          // [GM_KC][GM_LDA]
  double* Bs = sm + GM_KC * GM_LDA;         // [GM_KC][GM_LDB]
  double* Cs = sm;                          // [GM_TR][GM_LDC], aliases At / Bs after the K loop
  double* base = sm + GM_TR * GM_LDC;       // [GM_TN] run-covered base vector
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r0 = blockIdx.x * GM_TR, r1 = min(nRows, r0 + GM_TR);
  const int j0 = blockIdx.y * GM_TN, vc = min(GM_TN, vCols - j0);
  double c[2][8][2];
#pragma unroll
  for (int mt = 0; mt < 2; mt++)
#pragma unroll
    for (int nt = 0; nt < 8; nt++) c[mt][nt][0] = c[mt][nt][1] = 0.0;
  const int am = lane >> 2, ak = lane & 3;

  for (int k0 = 0; k0 < nDense; k0 += GM_KC) {
    // ---- stage: thread = (row, half of the 32 columns); lanes run along rows ----
    {
      const int r = tid & (GM_TR - 1), kh = tid >> 7;  // kh in {0, 1}: columns kh*16 .. +16
      const int row = r0 + r;
#pragma unroll 4
      for (int kk = 0; kk < 16; kk++) {
        const int kc = kh * 16 + kk;
        double v = 0.0;
        if (k0 + kc < nDense && row < nRows) {
          const DenseCol dc = dcols[k0 + kc];
          const DevGroup& g = groups[dc.group];
          if (g.type == GT_UNC) v = g.dense[(size_t)row * g.gCols + dc.j];
          else v = g.dict[(size_t)map_get(g.mapType, g.map, g.mapHi, row) * g.gCols + dc.j];
        }
        At[kc * GM_LDA + r] = v;
      }
      // V rows of these 32 dense columns
      for (int e = tid; e < GM_KC * GM_TN; e += GM_THREADS) {
        const int kc = e >> 6, n = e & 63;
        double v = 0.0;
        if (k0 + kc < nDense && n < vc) v = V[(size_t)dcols[k0 + kc].col * vCols + j0 + n];
        Bs[kc * GM_LDB + n] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < GM_KC; ks += 4) {
      double a[2];
#pragma unroll
      for (int mt = 0; mt < 2; mt++) a[mt] = At[(ks + ak) * GM_LDA + warp * 16 + mt * 8 + am];
#pragma unroll
      for (int nt = 0; nt < 8; nt++) {
        const double b = Bs[(ks + ak) * GM_LDB + nt * 8 + am];
#pragma unroll
        for (int mt = 0; mt < 2; mt++) dmma884(c[mt][nt][0], c[mt][nt][1], a[mt], b);
      }
    }
    __syncthreads();
  }

  // C fragment: row = lane >> 2, columns (lane & 3) * 2 + {0, 1}
  if (!hasSparse) {
#pragma unroll
    for (int mt = 0; mt < 2; mt++) {
      const int row = r0 + warp * 16 + mt * 8 + (lane >> 2);
      if (row >= r1) continue;
#pragma unroll
      for (int nt = 0; nt < 8; nt++)
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int n = nt * 8 + (lane & 3) * 2 + u;
          if (n < vc) out[(size_t)row * vCols + j0 + n] = c[mt][nt][u] + (constRow ? constRow[j0 + n] : 0.0);
        }
    }
    return;
  }
#pragma unroll
  for (int mt = 0; mt < 2; mt++)
#pragma unroll
    for (int nt = 0; nt < 8; nt++)
#pragma unroll
      for (int u = 0; u < 2; u++)
        Cs[(warp * 16 + mt * 8 + (lane >> 2)) * GM_LDC + nt * 8 + (lane & 3) * 2 + u] = c[mt][nt][u];
  if (tid < GM_TN) base[tid] = constRow && tid < vc ? constRow[j0 + tid] : 0.0;
  __syncthreads();
  // ---- sparse groups, one per warp at a time ----
  double b0 = 0.0, b1 = 0.0;  // this warp's share of the base vector: columns lane and lane + 32
  for (int gi = warp; gi < nGroups; gi += GM_THREADS / 32) {
    const DevGroup& g = groups[gi];
    if (g.type == GT_SDC) {
      const double* Pg = P + g.valOff * vCols + j0;
      // listed rows of the tile: decode 32 at a time, then the whole warp adds one table row per listed row
      sdc_walk_block(g, r0, r1, [&](int row, int e) {
        const int id = g.single ? 0 : map_get(g.mapType, g.map, g.mapHi, e);
        double* cr = Cs + (row - r0) * GM_LDC;
        const double* p = Pg + (size_t)id * vCols;
        for (int n = 0; n < vc; n++) atomicAdd(&cr[n], p[n]);
      });
    } else if (g.type == GT_RLE) {
      const double* Pg = P + g.valOff * vCols + j0;
      for (int64_t ri = g.runSkip[r0 / SKIP_ROWS]; ri < g.nRuns; ri++) {
        const RleRun run = g.runs[ri];
        if (run.start >= r1) break;
        const int a = max(run.start, r0), b = min(run.start + (int)run.len, r1);
        if (a >= b) continue;
        const double* p = Pg + (size_t)run.k * vCols;
        const double p0 = lane < vc ? p[lane] : 0.0, p1 = lane + 32 < vc ? p[lane + 32] : 0.0;
        if (a == r0 && b == r1) {  // the run covers the tile: one add to the base vector
          b0 += p0;
          b1 += p1;
        } else {
          for (int r = a; r < b; r++) {
            if (lane < vc) atomicAdd(&Cs[(r - r0) * GM_LDC + lane], p0);
            if (lane + 32 < vc) atomicAdd(&Cs[(r - r0) * GM_LDC + lane + 32], p1);
          }
        }
      }
    }
  }
  if (b0 != 0.0) atomicAdd(&base[lane], b0);
  if (b1 != 0.0) atomicAdd(&base[lane + 32], b1);
  __syncthreads();
  for (int e = tid; e < GM_TR * GM_TN; e += GM_THREADS) {
    const int r = e >> 6, n = e & 63;
    if (r0 + r < r1 && n < vc) out[(size_t)(r0 + r) * vCols + j0 + n] = Cs[r * GM_LDC + n] + base[n];
  }
}

// dictionary pre-aggregation for the groups that are added from tables (SDC, RLE)
__global__ void k_dict_times_v_sparse(const DevGroup* __restrict__ groups, const double* __restrict__ V, int vCols,
                                      double* __restrict__ P) {
  const DevGroup g = groups[blockIdx.x];
  if (g.type != GT_SDC && g.type != GT_RLE) return;
  const int64_t n = (int64_t)g.nVals * vCols;
  for (int64_t e = blockIdx.y * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.y * blockDim.x) {
    const int k = (int)(e / vCols), j = (int)(e - (int64_t)k * vCols);
    double s = 0;
    for (int h = 0; h < g.gCols; h++) s += g.dict[(size_t)k * g.gCols + h] * V[(size_t)g.cols[h] * vCols + j];
    P[(g.valOff + k) * vCols + j] = s;
  }
}

__global__ void k_const_times_v2(const double* __restrict__ constV, int nCols, const double* __restrict__ V, int vCols,
                                 double* __restrict__ constRow) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= vCols) return;
  double s = 0;
  for (int c = 0; c < nCols; c++) s += constV[c] * V[(size_t)c * vCols + j];
  constRow[j] = s;
}

// Builds (once per handle) the list of dense-operand columns.
static int64_t ensure_dense_cols(Matrix* m) {
  if (m->dDenseCols || m->denseColsBuilt) return CLA_OK;
  std::vector<DenseCol> dc;
  for (int gi = 0; gi < m->nDev; gi++) {
    const DevGroup& g = m->groups[gi];
    if (g.type != GT_DDC && g.type != GT_UNC) continue;
    std::vector<int32_t> cols(g.gCols);
    CLA_CUDA(cudaMemcpy(cols.data(), g.cols, cols.size() * 4, cudaMemcpyDeviceToHost));
    for (int j = 0; j < g.gCols; j++) dc.push_back(DenseCol{gi, j, cols[j], 0});
  }
  m->nDenseCols = (int)dc.size();
  m->denseColsBuilt = true;
  if (dc.empty()) return CLA_OK;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, dc.size() * sizeof(DenseCol));
  if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc dense column list: ") + cudaGetErrorString(e));
  m->allocs.push_back(p);
  CLA_CUDA(cudaMemcpy(p, dc.data(), dc.size() * sizeof(DenseCol), cudaMemcpyHostToDevice));
  m->dDenseCols = p;
  return CLA_OK;
}

int64_t launch_rmm_dmma(Matrix* m, const double* dV, int vCols, double* dOut, cudaStream_t s) {
  if (m->nRows == 0 || vCols == 0) return CLA_OK;
  int64_t rc;
  if ((rc = ensure_dense_cols(m)) < 0) return rc;
  const size_t pBytes = ((size_t)std::max<int64_t>(m->totalVals, 1) * vCols * sizeof(double) + 255) & ~(size_t)255;
  if ((rc = ensure_scratch(m, pBytes + (size_t)vCols * sizeof(double))) < 0) return rc;
  double* P = (double*)m->scratch;
  double* constRow = nullptr;
  int hasSparse = 0;
  int64_t maxE = 1;
  for (auto& g : m->groups)
    if (g.type == GT_SDC || g.type == GT_RLE) {
      hasSparse = 1;
      maxE = std::max<int64_t>(maxE, (int64_t)g.nVals * vCols);
    }
  if (hasSparse) {
    dim3 grid(m->nDev, (unsigned)std::max<int64_t>(1, std::min<int64_t>(64, (maxE + 255) / 256)));
    k_dict_times_v_sparse<<<grid, 256, 0, s>>>(m->dGroups, dV, vCols, P);
    m->stats.kernel_launches++;
  }
  if (m->hasConst) {
    constRow = (double*)((char*)m->scratch + pBytes);
    k_const_times_v2<<<(vCols + 127) / 128, 128, 0, s>>>(m->dConstV, m->nCols, dV, vCols, constRow);
    m->stats.kernel_launches++;
  }
  const size_t smem = std::max((size_t)(GM_KC * GM_LDA + GM_KC * GM_LDB), (size_t)(GM_TR * GM_LDC + GM_TN)) * sizeof(double);
  static bool attr = false;
  if (!attr) {
    CLA_CUDA(cudaFuncSetAttribute(k_rmm_dmma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr = true;
  }
  dim3 grid((m->nRows + GM_TR - 1) / GM_TR, (vCols + GM_TN - 1) / GM_TN);
  prof_begin(m, s);
  k_rmm_dmma<<<grid, GM_THREADS, smem, s>>>(m->dGroups, m->nDev, (const DenseCol*)m->dDenseCols, m->nDenseCols, m->nRows,
                                           dV, vCols, P, constRow, dOut, hasSparse);
  prof_end(m, s);
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

}  // namespace cla
