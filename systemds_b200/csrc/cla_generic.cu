// General product kernels: they accept every group type, any number of right-hand columns / left
// rows, and overlapping groups. The specialised kernels in cla_fast.cu take over for the shapes
// they cover; everything else runs here.
//
//   RMM  (CLALibRightMultBy.RMM, lib/CLALibRightMultBy.java:208-258)
//        1. k_dict_times_v : P_g = D_g * V[cols_g, :] for every dictionary group
//                            (ADictBasedColGroup.rightMultByMatrix, colgroup/ADictBasedColGroup.java:246-275)
//        2. k_rmm_vec_general : one right-hand column; a CTA owns a block of output rows and sums
//                            P_g[id_g(r)] over all groups, then adds constV * v (the decompress-and-sum of
//                            lib/CLALibDecompress.java:310-357). Wider right-hand sides run on the FP64
//                            tensor cores (cla_rmm_dmma.cu) or, for a few columns, once per column.
//   LMM  (CLALibLeftMultBy.LMM, lib/CLALibLeftMultBy.java:286-346)
//        1. k_lmm_preagg   : A_g[i, k] = sum of Yt[i, r] over rows r holding tuple k
//                            (APreAgg.preAggregateDense, colgroup/APreAgg.java:137)
//        2. k_lmm_post     : out[i, cols_g] += A_g[i, :] * D_g  (APreAgg.mmWithDictionary, :312-322)
//        3. k_lmm_unc      : uncompressed groups, direct product (ColGroupUncompressed.java:429-539)
//        4. k_lmm_const    : out += rowSums(Yt) (x) constV  (lib/CLALibLeftMultBy.java:530-629)
#include "cla_common.cuh"
#include <algorithm>
#include <climits>

namespace cla {

static inline int grid_for(int64_t n, int block, int cap = 148 * 16) {
  int64_t g = (n + block - 1) / block;
  return (int)std::max<int64_t>(1, std::min<int64_t>(g, cap));
}

// --------------------------------------------------------------------------------------------------
// P arena: [totalVals x vCols]
// --------------------------------------------------------------------------------------------------
__global__ void k_dict_times_v(const DevGroup* __restrict__ groups, const double* __restrict__ V, int vCols,
                               double* __restrict__ P, int skipFast) {
  const DevGroup g = groups[blockIdx.x];
  if (g.type == GT_UNC || (skipFast && g.inFast)) return;
  const int64_t n = (int64_t)g.nVals * vCols;
  for (int64_t e = blockIdx.y * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.y * blockDim.x) {
    const int k = (int)(e / vCols), j = (int)(e - (int64_t)k * vCols);
    double s = 0;
    for (int h = 0; h < g.gCols; h++) s += g.dict[(size_t)k * g.gCols + h] * V[(size_t)g.cols[h] * vCols + j];
    P[(g.valOff + k) * vCols + j] = s;
  }
}

// constRow[j] = sum_c constV[c] * V[c, j]
__global__ void k_const_times_v(const double* __restrict__ constV, int nCols, const double* __restrict__ V, int vCols,
                                double* __restrict__ constRow) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= vCols) return;
  double s = 0;
  for (int c = 0; c < nCols; c++) s += constV[c] * V[(size_t)c * vCols + j];
  constRow[j] = s;
}

// --------------------------------------------------------------------------------------------------
// X %*% v (one column) for every group type. A CTA owns one 1024-row block (the granularity of the skip
// indexes) and keeps its 1024 partial sums in shared memory. Every row's sum is formed in a fixed order, so a
// repeated call returns the same bits whatever else runs on the GPU:
//  1. dense-map groups in list order: a thread per row adds P_g[id];
//  2. uncompressed groups in list order: a warp per row, lanes along the dense row, shuffle reduction;
//  3. SDC and RLE groups in list order, eight at a time: warp w writes the values group 8 i + w contributes to the
//     block's rows into its own row of a staging tile (SDC: warp-scan decode of the delta stream from the block's
//     skip entry; RLE: the runs that reach into the block), then the thread that owns a row adds the eight staged
//     values in group order. No atomics: each staging row has one writer, each sum one owner.
//  4. the constant part.
// (The reference sums a row's groups in list order and the constants last, lib/CLALibDecompress.java:427-434;
// here the order is by kind, then list order.)
// --------------------------------------------------------------------------------------------------
constexpr int RV_THREADS = 256;
constexpr int RV_WARPS = RV_THREADS / 32;
constexpr size_t RV_SMEM = (size_t)(RV_WARPS + 1) * SKIP_ROWS * sizeof(double);
// LISTS: the SDC / RLE contributions come from the row-major work lists (8-row steps, 64-row windows) instead of the
// rounds of step 3: a thread owns one step of the block and applies its items in list order to its own eight sums,
// a thread per window sums the runs that cover the window. No staging tile, two shared-memory updates per listed
// row instead of sixteen per row and round.
constexpr size_t RV_SMEM_LISTS = (size_t)(2 * SKIP_ROWS + 16) * sizeof(double);
template <bool LISTS>
__global__ void __launch_bounds__(RV_THREADS)
k_rmm_vec_general(const DevGroup* __restrict__ groups, const int32_t* __restrict__ ddcIdx, int nDdc,
                  const int32_t* __restrict__ uncIdx, int nUnc, const int32_t* __restrict__ sparseIdx, int nSparse, int nRows, const double* __restrict__ P, const double* __restrict__ v,
                  const double* __restrict__ constRow, double* __restrict__ out, int afterFast,
                  const SpItem* __restrict__ stepItems, const uint32_t* __restrict__ stepPtr, int64_t nStepPtr,
                  const SpItem* __restrict__ winItems, const uint32_t* __restrict__ winPtr, int64_t nWinPtr) {
  extern __shared__ __align__(16) double rvsm[];
  double* acc = rvsm;                  // [SKIP_ROWS]
  double* stage = rvsm + SKIP_ROWS;    // [RV_WARPS][SKIP_ROWS]; LISTS: sums of the steps [8][128], then 16 window sums
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r0 = blockIdx.x * SKIP_ROWS, r1 = min(nRows, r0 + SKIP_ROWS);
  for (int i = tid; i < SKIP_ROWS; i += RV_THREADS) acc[i] = 0.0;
  __syncthreads();
  // dense-map groups (list order; after the specialised kernels only those they left): a thread owns rows tid, tid + 256, ...
  for (int i = 0; i < nDdc; i++) {
    const DevGroup& g = groups[ddcIdx[i]];
    const double* Pg = P + g.valOff;
    for (int r = r0 + tid; r < r1; r += RV_THREADS) acc[r - r0] += Pg[map_get(g.mapType, g.map, g.mapHi, r)];
  }
  __syncthreads();
  // uncompressed groups: a warp owns rows warp, warp + 8, ...; lanes along the dense row, two columns each per pass,
  // four rows in flight (their loads are issued before the first of the four shuffle reductions)
  for (int i = 0; i < nUnc; i++) {
    const DevGroup& g = groups[uncIdx[i]];
    const int gc = g.gCols;
    const double* __restrict__ dense = g.dense;
    for (int cb = 0; cb < gc; cb += 64) {
      const int ca = cb + lane, cc = cb + 32 + lane;
      const double va = ca < gc ? v[g.cols[ca]] : 0.0, vb = cc < gc ? v[g.cols[cc]] : 0.0;
      for (int rb = r0 + warp * 4; rb < r1; rb += RV_WARPS * 4) {
        double sum[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int r = rb + q;
          const double* row = dense + (size_t)r * gc;
          const double xa = (r < r1 && ca < gc) ? row[ca] : 0.0, xb = (r < r1 && cc < gc) ? row[cc] : 0.0;
          sum[q] = xa * va + xb * vb;
        }
#pragma unroll
        for (int q = 0; q < 4; q++)
          for (int d = 16; d; d >>= 1) sum[q] += __shfl_down_sync(0xffffffffu, sum[q], d);
        if (lane == 0) {
#pragma unroll
          for (int q = 0; q < 4; q++)
            if (rb + q < r1) acc[rb + q - r0] += sum[q];
        }
      }
    }
  }
  if (nUnc) __syncthreads();
  if (LISTS) {
    constexpr int NSTEP = SKIP_ROWS / G3_STEP, NWIN = SKIP_ROWS / G3_WIN;  // 128 steps, 16 windows per block
    double* sacc = stage;                 // row i of step t at [i * NSTEP + t]: neighbouring threads, neighbouring words
    double* wbase = stage + SKIP_ROWS;    // [NWIN]
    for (int i = tid; i < SKIP_ROWS; i += RV_THREADS) sacc[i] = 0.0;
    __syncthreads();
    if (tid < NWIN) {  // runs that cover a whole window
      const int64_t w = (int64_t)blockIdx.x * NWIN + tid;
      const uint32_t p0 = winPtr[min(w, nWinPtr - 1)], p1 = winPtr[min(w + 1, nWinPtr - 1)];
      double sum = 0.0;
      for (uint32_t i = p0; i < p1; i++) sum += P[winItems[i].prow];
      wbase[tid] = sum;
    } else if (tid >= RV_THREADS - NSTEP) {  // listed rows and run pieces of one 8-row step, in list order
      const int t = tid - (RV_THREADS - NSTEP);
      const int64_t st = (int64_t)blockIdx.x * NSTEP + t;
      const uint32_t p0 = stepPtr[min(st, nStepPtr - 1)], p1 = stepPtr[min(st + 1, nStepPtr - 1)];
      SpItem e = p0 < p1 ? stepItems[p0] : SpItem{0, 0};
      for (uint32_t i = p0; i < p1; i++) {
        const SpItem nxt = i + 1 < p1 ? stepItems[i + 1] : SpItem{0, 0};  // next item in flight during this one's table read
        const double p = P[e.prow];
        const int ra = e.rows & 0xFF, rb = (e.rows >> 8) & 0xFF;
        for (int r = ra; r < rb; r++) sacc[r * NSTEP + t] += p;
        e = nxt;
      }
    }
    __syncthreads();
    const double c0 = (constRow != nullptr && !afterFast) ? constRow[0] : 0.0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int rr = tid * 4 + i, r = r0 + rr;
      if (r < r1) {
        const double val = ((acc[rr] + sacc[(rr & 7) * NSTEP + (rr >> 3)]) + wbase[rr >> 6]) + c0;
        out[r] = afterFast ? out[r] + val : val;
      }
    }
    return;
  }
  // SDC / RLE groups, eight per round. From here on thread t owns rows 4 t .. 4 t + 3.
  double a4[4];
  {
    const double2 lo = *(const double2*)&acc[tid * 4], hi = *(const double2*)&acc[tid * 4 + 2];
    a4[0] = lo.x, a4[1] = lo.y, a4[2] = hi.x, a4[3] = hi.y;
  }
  double* mine = stage + warp * SKIP_ROWS;
  for (int s0 = 0; s0 < nSparse; s0 += RV_WARPS) {
    const int si = s0 + warp;
    if (si < nSparse) {
      double2* m2 = (double2*)mine;
      for (int i = lane; i < SKIP_ROWS / 2; i += 32) m2[i] = make_double2(0.0, 0.0);
      __syncwarp();
      const DevGroup& g = groups[sparseIdx[si]];
      const double* Pg = P + g.valOff;
      if (g.type == GT_SDC) {
        sdc_walk_block(g, r0, r1, [&](int row, int e) {
          mine[row - r0] = Pg[g.single ? 0 : map_get(g.mapType, g.map, g.mapHi, e)];
        });
      } else {  // RLE: a run writes its value to each of its rows (colgroup/ColGroupRLE.java:104-141)
        for (int64_t ri = g.runSkip[blockIdx.x]; ri < g.nRuns; ri++) {
          const RleRun run = g.runs[ri];
          if (run.start >= r1) break;
          const int a = max(run.start, r0), b = min(run.start + (int)run.len, r1);
          const double p = Pg[run.k];
          for (int i = a + lane; i < b; i += 32) mine[i - r0] = p;
        }
      }
    }
    __syncthreads();
    const int nw = min(RV_WARPS, nSparse - s0);
    for (int w = 0; w < nw; w++) {
      const double2 lo = *(const double2*)&stage[w * SKIP_ROWS + tid * 4];
      const double2 hi = *(const double2*)&stage[w * SKIP_ROWS + tid * 4 + 2];
      // rows a group does not list hold 0.0 here; adding it changes nothing
      a4[0] += lo.x, a4[1] += lo.y, a4[2] += hi.x, a4[3] += hi.y;
    }
    __syncthreads();
  }
  const double c0 = (constRow != nullptr && !afterFast) ? constRow[0] : 0.0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int r = r0 + tid * 4 + i;
    if (r < r1) {
      const double val = a4[i] + c0;
      out[r] = afterFast ? out[r] + val : val;
    }
  }
}

// SDC groups with listed rows and RLE groups with runs, in list order (built once per handle)
int64_t ensure_sparse_list(Matrix* m) {
  if (m->sparseListBuilt) return CLA_OK;
  std::vector<int32_t> sparse, ddc, ddcRest, unc;
  for (int gi = 0; gi < m->nDev; gi++) {
    const DevGroup& g = m->groups[gi];
    if ((g.type == GT_SDC && g.nOff > 0) || (g.type == GT_RLE && g.nRuns > 0)) sparse.push_back(gi);
    if (g.type == GT_DDC) {
      ddc.push_back(gi);
      if (!g.inFast) ddcRest.push_back(gi);
    }
    if (g.type == GT_UNC) unc.push_back(gi);
  }
  auto up = [&](const std::vector<int32_t>& idx, int32_t** d) -> int64_t {
    if (idx.empty()) return CLA_OK;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, idx.size() * sizeof(int32_t));
    if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc group list: ") + cudaGetErrorString(e));
    m->allocs.push_back(p);
    CLA_CUDA(cudaMemcpy(p, idx.data(), idx.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
    *d = (int32_t*)p;
    return CLA_OK;
  };
  int64_t rc;
  if ((rc = up(sparse, &m->dSparseIdx)) < 0 || (rc = up(ddc, &m->dDdcIdx)) < 0 || (rc = up(ddcRest, &m->dDdcRestIdx)) < 0 ||
      (rc = up(unc, &m->dUncIdx)) < 0)
    return rc;
  m->nSparse = (int)sparse.size();
  m->nDdc = (int)ddc.size();
  m->nDdcRest = (int)ddcRest.size();
  m->nUnc = (int)unc.size();
  m->sparseListBuilt = true;
  return CLA_OK;
}

int64_t launch_rmm(Matrix* m, const double* dV, int vCols, double* dOut, cudaStream_t s, bool afterFast) {
  if (m->nRows == 0 || vCols == 0) return CLA_OK;
  if (vCols != 1) return fail(CLA_ERR_UNSUPPORTED, "rmm: the general kernel takes one right-hand column");
  if (afterFast) {  // nothing left for this pass if the specialised kernels covered every group
    bool rest = false;
    for (auto& g : m->groups) rest |= !g.inFast;
    if (!rest) return CLA_OK;
  }
  int64_t rc;
  if ((rc = ensure_sparse_list(m)) < 0) return rc;
  const size_t pBytes = (size_t)std::max<int64_t>(m->totalVals, 1) * sizeof(double);
  const size_t cOff = (pBytes + 255) & ~(size_t)255;
  if ((rc = ensure_scratch(m, cOff + sizeof(double))) < 0) return rc;
  double* P = (double*)m->scratch;
  double* constRow = nullptr;
  if (m->nDev > 0) {
    int maxE = 1;
    for (auto& g : m->groups) maxE = std::max<int64_t>(maxE, (int64_t)g.nVals);
    dim3 grid(m->nDev, std::max(1, std::min(64, (maxE + 255) / 256)));
    k_dict_times_v<<<grid, 256, 0, s>>>(m->dGroups, dV, 1, P, afterFast ? 1 : 0);
    m->stats.kernel_launches++;
  }
  if (m->hasConst && !afterFast) {
    constRow = (double*)((char*)m->scratch + cOff);
    k_const_times_v<<<1, 128, 0, s>>>(m->dConstV, m->nCols, dV, 1, constRow);
    m->stats.kernel_launches++;
  }
  static bool attrSet[64] = {};  // per device: function attributes belong to the device's context
  bool& attr = attrSet[m->device & 63];
  if (!attr) {
    CLA_CUDA(cudaFuncSetAttribute(k_rmm_vec_general<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RV_SMEM));
    attr = true;
  }
  // matrices with many listed rows: the row-major work lists (shared with the tensor-core right product), built once
  bool lists = false;
  if (m->nSparse > 0 && m->nRows >= 4 * SKIP_ROWS) {
    if ((rc = ensure_sparse_lists(m, s)) < 0) return rc;
    lists = m->spListsOk && m->dStepPtr != nullptr;
  }
  const int32_t* ddcIdx = afterFast ? m->dDdcRestIdx : m->dDdcIdx;
  const int nDdc = afterFast ? m->nDdcRest : m->nDdc;
  prof_begin(m, s);
  const unsigned grid = (unsigned)((m->nRows + SKIP_ROWS - 1) / SKIP_ROWS);
  if (lists)
    k_rmm_vec_general<true><<<grid, RV_THREADS, RV_SMEM_LISTS, s>>>(
        m->dGroups, ddcIdx, nDdc, m->dUncIdx, m->nUnc, m->dSparseIdx, m->nSparse, m->nRows, P, dV, constRow, dOut, afterFast ? 1 : 0,
        (const SpItem*)m->dStepItems, m->dStepPtr, m->nStepPtr, (const SpItem*)m->dWinItems, m->dWinPtr, m->nWinPtr);
  else
    k_rmm_vec_general<false><<<grid, RV_THREADS, RV_SMEM, s>>>(m->dGroups, ddcIdx, nDdc, m->dUncIdx, m->nUnc, m->dSparseIdx, m->nSparse, m->nRows, P, dV,
                                                             constRow, dOut, afterFast ? 1 : 0, nullptr, nullptr, 0, nullptr,
                                                             nullptr, 0);
  prof_end(m, s);
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

// --------------------------------------------------------------------------------------------------
// X %*% V kept compressed (CLALibRightMultBy.RMMOverlapping, lib/CLALibRightMultBy.java:157-201): every dictionary
// group of X becomes a group over all vCols result columns that keeps its index structure (the maps, offset
// streams and run lists are shared with X, not copied) and gets the dictionary P_g = D_g * V[cols_g, :]
// (ADictBasedColGroup.rightMultByMatrix, colgroup/ADictBasedColGroup.java:246-275); an uncompressed group becomes the
// uncompressed product of its block (colgroup/ColGroupUncompressed.java, rightMultByMatrix); the constants become
// constV * V (addConstant, :203-206). The result is an overlapping block: its cells are the sums over the groups.
// --------------------------------------------------------------------------------------------------
__global__ void k_unc_times_v(const double* __restrict__ dense, int gCols, const int32_t* __restrict__ cols, int64_t nRows,
                              const double* __restrict__ V, int vCols, double* __restrict__ out) {
  const int64_t n = nRows * vCols;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / vCols;
    const int j = (int)(e - r * vCols);
    double s = 0;
    for (int c = 0; c < gCols; c++) s += dense[r * gCols + c] * V[(size_t)cols[c] * vCols + j];
    out[e] = s;
  }
}
__global__ void k_iota_cols(int32_t* p, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = i;
}

int64_t make_overlapping(Matrix* m, Matrix* child, const double* dV, int vCols, cudaStream_t s) {
  auto dalloc = [&](void** p, size_t bytes) -> int64_t {
    *p = nullptr;
    cudaError_t e = cudaMalloc(p, std::max<size_t>(bytes, 16));
    if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc overlapping result: ") + cudaGetErrorString(e));
    child->allocs.push_back(*p);
    child->deviceBytes += (int64_t)bytes;
    return CLA_OK;
  };
  int64_t rc;
  child->nRows = m->nRows;
  child->nCols = vCols;
  child->overlapping = true;
  child->multiCover = true;
  child->colSrcValid = false;
  child->device = m->device;
  if ((rc = init_device_state(child)) < 0) return rc;
  void *P = nullptr, *iota = nullptr, *cst = nullptr;
  if ((rc = dalloc(&P, (size_t)std::max<int64_t>(m->totalVals, 1) * vCols * sizeof(double))) < 0) return rc;
  if ((rc = dalloc(&iota, (size_t)std::max(vCols, 1) * sizeof(int32_t))) < 0) return rc;
  if ((rc = dalloc(&cst, (size_t)std::max(vCols, 1) * sizeof(double))) < 0) return rc;
  if (vCols > 0) k_iota_cols<<<(vCols + 255) / 256, 256, 0, s>>>((int32_t*)iota, vCols);
  if (m->nDev > 0 && vCols > 0) {
    int64_t maxE = 1;
    for (auto& g : m->groups) maxE = std::max<int64_t>(maxE, (int64_t)g.nVals * vCols);
    dim3 grid(m->nDev, (unsigned)std::max<int64_t>(1, std::min<int64_t>(64, (maxE + 255) / 256)));
    k_dict_times_v<<<grid, 256, 0, s>>>(m->dGroups, dV, vCols, (double*)P, 0);
  }
  child->constV.assign(vCols, 0.0);
  if (m->hasConst && vCols > 0) {
    k_const_times_v<<<(vCols + 127) / 128, 128, 0, s>>>(m->dConstV, m->nCols, dV, vCols, (double*)cst);
    CLA_CUDA(cudaMemcpyAsync(child->constV.data(), cst, (size_t)vCols * sizeof(double), cudaMemcpyDeviceToHost, s));
  } else
    CLA_CUDA(cudaMemsetAsync(cst, 0, (size_t)std::max(vCols, 1) * sizeof(double), s));
  child->dConstV = (double*)cst;
  // the groups: same index structures, new dictionaries / dense blocks, every group over all result columns
  child->groups.clear();
  child->hg.clear();
  child->regToDev.clear();
  for (int gi = 0; gi < m->nDev; gi++) {
    DevGroup g = m->groups[gi];
    HostGroup hg;  // the record kept after finalize: type, width, number of tuples
    hg.type = g.origType;
    hg.cols.resize(vCols);
    for (int j = 0; j < vCols; j++) hg.cols[j] = j;
    hg.nVals = g.origType == GT_OLE ? g.nVals - 1 : g.nVals;
    if (g.type == GT_UNC) {
      void* d = nullptr;
      if ((rc = dalloc(&d, (size_t)m->nRows * vCols * sizeof(double))) < 0) return rc;
      if ((int64_t)m->nRows * vCols > 0)
        k_unc_times_v<<<grid_for((int64_t)m->nRows * vCols, 256), 256, 0, s>>>(g.dense, g.gCols, g.cols, m->nRows, dV, vCols, (double*)d);
      g.dense = (const double*)d;
    } else {
      g.dict = g.dictRaw = (const double*)P + (size_t)g.valOff * vCols;
    }
    g.gCols = vCols;
    g.cols = (const int32_t*)iota;
    g.inFast = 0;
    child->regToDev.push_back((int)child->groups.size());
    child->groups.push_back(g);
    child->hg.push_back(std::move(hg));
  }
  child->nDev = (int)child->groups.size();
  child->totalVals = m->totalVals;
  void* dg = nullptr;
  if ((rc = dalloc(&dg, std::max<size_t>(child->groups.size(), 1) * sizeof(DevGroup))) < 0) return rc;
  if (!child->groups.empty())
    CLA_CUDA(cudaMemcpyAsync(dg, child->groups.data(), child->groups.size() * sizeof(DevGroup), cudaMemcpyHostToDevice, s));
  child->dGroups = (DevGroup*)dg;
  void* cs = nullptr;  // column -> group table: unused for overlapping blocks, but allocated like everywhere else
  if ((rc = dalloc(&cs, (size_t)std::max(vCols, 1) * 2 * sizeof(int32_t))) < 0) return rc;
  CLA_CUDA(cudaMemsetAsync(cs, 0xFF, (size_t)std::max(vCols, 1) * 2 * sizeof(int32_t), s));
  child->dColSrc = (int32_t*)cs;
  CLA_CUDA(cudaStreamSynchronize(s));
  CLA_CUDA(cudaGetLastError());
  child->hasConst = false;
  for (double x : child->constV) child->hasConst |= (x != 0.0);
  child->colMin.assign(vCols, 0.0);  // extrema of an overlapping block are taken from decompressed rows
  child->colMax.assign(vCols, 0.0);
  child->indexBytes = (int64_t)std::max<int64_t>(m->totalVals, 1) * vCols * 8;
  child->stats.n_cols = vCols;
  child->stats.n_groups = (int64_t)child->hg.size();
  child->stats.device_bytes = child->deviceBytes;
  child->stats.index_bytes = child->indexBytes;
  child->finalized = true;
  return CLA_OK;
}

// --------------------------------------------------------------------------------------------------
// decompress = RMM with V = I restricted to the group's own columns: out[r, cols_g] += D_g[id_g(r), :]
// One launch per group keeps the reference's "groups in list order" summation
// (lib/CLALibDecompress.java:427-434) without atomics.
// --------------------------------------------------------------------------------------------------
__global__ void k_decomp_init(double* __restrict__ out, const double* __restrict__ constV, int64_t nRows, int nCols) {
  const int64_t n = nRows * nCols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = constV ? constV[i % nCols] : 0.0;
}
// rows [r0, r1); out points at row r0
__global__ void k_decomp_dense(DevGroup g, double* __restrict__ out, int r0, int r1, int nCols) {
  const int64_t n = (int64_t)(r1 - r0) * g.gCols;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / g.gCols;
    const int c = (int)(e - r * g.gCols);
    double v;
    if (g.type == GT_UNC) v = g.dense[(size_t)(r0 + r) * g.gCols + c];
    else v = g.dict[(size_t)map_get(g.mapType, g.map, g.mapHi, r0 + r) * g.gCols + c];
    out[r * nCols + g.cols[c]] += v;
  }
}
__global__ void k_decomp_sdc(DevGroup g, double* __restrict__ out, int r0, int r1, int nCols) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int rb = r0 + warp * SKIP_ROWS;
  if (rb >= r1) return;
  const int re = min(r1, rb + SKIP_ROWS);
  sdc_walk_block(g, rb, re, [&](int row, int e) {
    const int id = g.single ? 0 : map_get(g.mapType, g.map, g.mapHi, e);
    for (int c = 0; c < g.gCols; c++) out[(size_t)(row - r0) * nCols + g.cols[c]] += g.dict[(size_t)id * g.gCols + c];
  });
}
__global__ void k_decomp_rle(DevGroup g, double* __restrict__ out, int r0, int r1, int nCols) {
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nWarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int64_t ri = g.runSkip[r0 / SKIP_ROWS] + warp; ri < g.nRuns; ri += nWarps) {
    const RleRun r = g.runs[ri];
    if (r.start >= r1) break;
    const int a = max(r.start, r0), b = min(r.start + (int)r.len, r1);
    for (int i = a + lane; i < b; i += 32)
      for (int c = 0; c < g.gCols; c++) out[(size_t)(i - r0) * nCols + g.cols[c]] += g.dict[(size_t)r.k * g.gCols + c];
  }
}

// Decompress of a block whose columns each belong to at most one group, every group type, one pass: a CTA owns
// 128 rows x 32 columns and builds them in shared memory, a warp per column (two columns each) with lanes along the
// rows -- a dense-map column reads four consecutive ids per lane (one 128-byte line per warp for byte maps), an SDC
// column fills its constant and then scatters the listed rows (warp-scan decode from the skip entry), an RLE column
// fills its runs -- and then writes the tile out a row per warp instruction, 256 contiguous bytes per row.
// Uncompressed columns skip the tile: adjacent columns are adjacent in memory, so the write-out loop reads them.
// Every output cell is written exactly once; nothing is read back. (Measured alternatives, both slower: a 256 x 8
// tile, whose 64-byte output pieces lie 4 KB apart; persistent CTAs that keep their columns' dictionaries in shared
// memory -- the kernel is bound by the latency of its load -> lookup -> store chain, which many small CTAs hide
// better than few large ones.)
constexpr int DB_COLS = 32;
constexpr int DB_ROWS = 128;
constexpr int DB_LD = DB_ROWS + 1;   // column stride of the tile (odd: the row-wise read of the write-out is conflict free)
// position of tile row r inside its column: the four rows of a lane go to four different 32-row groups, so a warp's
// store of one of them is contiguous
__device__ __forceinline__ int db_pos(int r) { return (r & 3) * 32 + (r >> 2); }
constexpr int DB_WARPS = 16;  // two columns per warp (measured 4 / 8 / 16 / 32 warps on 1M x 500 mixed: 2.54 / 2.11 / 1.87 / 2.07 ms)
__global__ void __launch_bounds__(DB_WARPS * 32)
k_decomp_block(const DevGroup* __restrict__ groups, const int32_t* __restrict__ colSrc, const double* __restrict__ constV,
               double* __restrict__ out, int r0, int r1, int nCols, int exactSdc) {
  extern __shared__ double dtile[];  // [DB_COLS][DB_LD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rb = r0 + blockIdx.x * DB_ROWS, re = min(r1, rb + DB_ROWS), nr = re - rb;
  const int c0 = blockIdx.y * DB_COLS, nc = min(DB_COLS, nCols - c0);
  __shared__ const double* uncSrc[DB_COLS];  // uncompressed columns: first value of the column (+ constant below)
  __shared__ int uncStride[DB_COLS];
  __shared__ double uncCst[DB_COLS];
  if (tid < DB_COLS) {
    uncSrc[tid] = nullptr;
    if (tid < nc) {
      const int gi = colSrc[2 * (c0 + tid)];
      if (gi >= 0 && groups[gi].type == GT_UNC) {
        uncSrc[tid] = groups[gi].dense + colSrc[2 * (c0 + tid) + 1];
        uncStride[tid] = groups[gi].gCols;
        uncCst[tid] = constV ? constV[c0 + tid] : 0.0;
      }
    }
  }
  for (int cw = warp; cw < nc; cw += DB_WARPS) {
    const int c = c0 + cw;
    const int gi = colSrc[2 * c];
    const double cst = constV ? constV[c] : 0.0;
    double* col = dtile + cw * DB_LD;
    if (gi < 0) {
      for (int rr = lane; rr < nr; rr += 32) col[db_pos(rr)] = cst;
    } else {
      const DevGroup& g = groups[gi];
      const int j = colSrc[2 * c + 1], gc = g.gCols;
      const double* dict = g.dict + j;
      if (g.type == GT_DDC) {
        const int mt = g.mapType;
        // four consecutive rows per lane; all ids are loaded before the first dictionary read that needs one
        int id[4];
        const int rr0 = lane * 4;
        if ((mt == CLA_MAP_UBYTE || mt == CLA_MAP_BYTE) && nr == DB_ROWS) {
          const uint32_t w = __ldg((const uint32_t*)((const uint8_t*)g.map + rb) + lane);  // rb is a multiple of 128
#pragma unroll
          for (int u = 0; u < 4; u++) id[u] = (w >> (8 * u)) & 0xFF;
        } else if (mt == CLA_MAP_CHAR && nr == DB_ROWS) {
          const uint2 w = __ldg((const uint2*)((const uint16_t*)g.map + rb) + lane);  // four 16-bit ids per lane
          id[0] = w.x & 0xFFFF;
          id[1] = w.x >> 16;
          id[2] = w.y & 0xFFFF;
          id[3] = w.y >> 16;
        } else {
#pragma unroll
          for (int u = 0; u < 4; u++) id[u] = rr0 + u < nr ? map_get(mt, g.map, g.mapHi, rb + rr0 + u) : 0;
        }
        double v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = dict[(size_t)id[u] * gc];
#pragma unroll
        for (int u = 0; u < 4; u++)
          if (rr0 + u < nr) col[u * 32 + lane] = cst + v[u];  // = db_pos(rr0 + u)
      } else if (g.type == GT_SDC) {
        for (int rr = lane; rr < nr; rr += 32) col[db_pos(rr)] = cst;
        __syncwarp();
        // exactSdc: the column belongs to this group alone, so its constant is exactly the group's default tuple and
        // a listed row holds the registered value itself (the reference writes d, lib/CLALibDecompress.java:310-357)
        const double* raw = g.dictRaw + j;
        sdc_walk_block(g, rb, re, [&](int row, int e) {
          const int id = g.single ? 0 : map_get(g.mapType, g.map, g.mapHi, e);
          col[db_pos(row - rb)] = exactSdc ? raw[(size_t)id * gc] : cst + dict[(size_t)id * gc];
        });
      } else if (g.type == GT_RLE) {
        for (int rr = lane; rr < nr; rr += 32) col[db_pos(rr)] = cst;
        __syncwarp();
        for (int64_t ri = g.runSkip[rb / SKIP_ROWS]; ri < g.nRuns; ri++) {
          const RleRun run = g.runs[ri];
          if (run.start >= re) break;
          const int a = max(run.start, rb), b = min(run.start + (int)run.len, re);
          const double v = cst + dict[(size_t)run.k * gc];
          for (int i = a + lane; i < b; i += 32) col[db_pos(i - rb)] = v;
        }
      }
    }
  }
  __syncthreads();
  // a row per warp instruction: lane = column of the tile
  if (lane < nc) {
    const double* us = uncSrc[lane];  // this lane's column: read once, not per row
    const size_t ustride = us ? (size_t)uncStride[lane] : 0;
    const double ucst = us ? uncCst[lane] : 0.0;
    const double* tcol = dtile + lane * DB_LD;
    double* o = out + (size_t)(rb - r0) * nCols + c0 + lane;
    for (int rr = warp; rr < nr; rr += DB_WARPS)
      o[(size_t)rr * nCols] = us ? ucst + us[(size_t)(rb + rr) * ustride] : tcol[db_pos(rr)];
  }
}

// r0 must be a multiple of SKIP_ROWS
int64_t launch_decompress_range(Matrix* m, int r0, int r1, double* dOut, cudaStream_t s) {
  const int64_t n = (int64_t)(r1 - r0) * m->nCols;
  if (n <= 0) return CLA_OK;
  if (m->colSrcValid) {  // no column held by two groups: one pass, every cell written once
    const int64_t rf = fast_decompress(m, r0, r1, dOut, s);  // byte-map matrices: straight from the column-per-lane layout
    if (rf != 0) return rf < 0 ? rf : CLA_OK;
    const size_t smem = (size_t)DB_COLS * DB_LD * sizeof(double);
    static bool attrSet[64] = {};  // per device: function attributes belong to the device's context
    bool& attr = attrSet[m->device & 63];
    if (!attr) {
      CLA_CUDA(cudaFuncSetAttribute(k_decomp_block, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      attr = true;
    }
    dim3 grid((r1 - r0 + DB_ROWS - 1) / DB_ROWS, (m->nCols + DB_COLS - 1) / DB_COLS);
    k_decomp_block<<<grid, DB_WARPS * 32, smem, s>>>(m->dGroups, m->dColSrc, m->hasConst ? m->dConstV : nullptr, dOut, r0, r1, m->nCols,
                                           m->multiCover ? 0 : 1);
    m->stats.kernel_launches++;
    CLA_CUDA(cudaGetLastError());
    return CLA_OK;
  }
  // overlapping groups: constants first, then every group adds its values (the reference's list-order summation)
  k_decomp_init<<<grid_for(n, 256), 256, 0, s>>>(dOut, m->hasConst ? m->dConstV : nullptr, r1 - r0, m->nCols);
  m->stats.kernel_launches++;
  for (auto& g : m->groups) {
    if (g.type == GT_DDC || g.type == GT_UNC)
      k_decomp_dense<<<grid_for((int64_t)(r1 - r0) * g.gCols, 256), 256, 0, s>>>(g, dOut, r0, r1, m->nCols);
    else if (g.type == GT_SDC) {
      const int nb = (r1 - r0 + SKIP_ROWS - 1) / SKIP_ROWS;
      k_decomp_sdc<<<(nb * 32 + 255) / 256, 256, 0, s>>>(g, dOut, r0, r1, m->nCols);
    } else if (g.type == GT_RLE && g.nRuns)
      k_decomp_rle<<<64, 256, 0, s>>>(g, dOut, r0, r1, m->nCols);
    m->stats.kernel_launches++;
  }
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

int64_t launch_decompress(Matrix* m, double* dOut, cudaStream_t s) {
  return launch_decompress_range(m, 0, m->nRows, dOut, s);
}

// --------------------------------------------------------------------------------------------------
// LMM
// --------------------------------------------------------------------------------------------------
constexpr int LMM_THREADS = 256;
constexpr int LMM_QT = 4;                 // left rows per pass (the reference's rowBlockSize)
constexpr int LMM_HIST_MAX = 6144;        // doubles of shared histogram (48 KB)

// grid: (row chunks, dictionary groups, q tiles). A: [totalVals x q]
__global__ void __launch_bounds__(LMM_THREADS)
k_lmm_preagg(const DevGroup* __restrict__ groups, int nRows, int rowsPerChunk, const double* __restrict__ Yt, int q,
             double* __restrict__ A, int skipFast, int skipSparse) {
  __shared__ double hist[LMM_HIST_MAX];
  const DevGroup& g = groups[blockIdx.y];
  if (g.type == GT_UNC || (skipFast && g.inFast)) return;
  if (skipSparse && (g.type == GT_SDC || g.type == GT_RLE)) return;  // taken from the row-major work lists (k_lmm_lists)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ra = blockIdx.x * rowsPerChunk, rb = min(nRows, ra + rowsPerChunk);
  if (ra >= rb) return;
  const int q0 = blockIdx.z * LMM_QT, qt = min(LMM_QT, q - q0);
  const int nv = g.nVals;
  const bool useShared = (int64_t)nv * qt <= LMM_HIST_MAX;
  double* Ag = A + g.valOff * q;
  if (useShared) {
    for (int e = tid; e < nv * qt; e += LMM_THREADS) hist[e] = 0.0;
    __syncthreads();
  }
  auto add = [&](int id, int i, double v) {
    if (useShared) atomicAdd(&hist[i * nv + id], v);
    else atomicAdd(&Ag[(size_t)id * q + q0 + i], v);
  };
  if (g.type == GT_DDC) {
    for (int r = ra + tid; r < rb; r += LMM_THREADS) {
      const int id = map_get(g.mapType, g.map, g.mapHi, r);
      for (int i = 0; i < qt; i++) add(id, i, Yt[(size_t)(q0 + i) * nRows + r]);
    }
  } else if (g.type == GT_SDC) {
    for (int b = ra + warp * SKIP_ROWS; b < rb; b += (LMM_THREADS / 32) * SKIP_ROWS) {
      sdc_walk_block(g, b, min(rb, b + SKIP_ROWS), [&](int row, int e) {
        const int id = g.single ? 0 : map_get(g.mapType, g.map, g.mapHi, e);
        for (int i = 0; i < qt; i++) add(id, i, Yt[(size_t)(q0 + i) * nRows + row]);
      });
    }
  } else if (g.type == GT_RLE) {
    // one warp per run: sum the left values over the run, then one add per left row
    for (int64_t ri = g.runSkip[ra / SKIP_ROWS] + warp; ri < g.nRuns; ri += LMM_THREADS / 32) {
      const RleRun run = g.runs[ri];
      if (run.start >= rb) break;
      const int a = max(run.start, ra), b = min(run.start + (int)run.len, rb);
      for (int i = 0; i < qt; i++) {
        double sum = 0;
        for (int r = a + lane; r < b; r += 32) sum += Yt[(size_t)(q0 + i) * nRows + r];
        for (int d = 16; d; d >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, d);
        if (lane == 0 && a < b) add(run.k, i, sum);
      }
    }
  }
  if (useShared) {
    __syncthreads();
    for (int e = tid; e < nv * qt; e += LMM_THREADS) {
      const double v = hist[e];
      if (v != 0.0) {
        const int i = e / nv, id = e - i * nv;
        atomicAdd(&Ag[(size_t)id * q + q0 + i], v);
      }
    }
  }
}

// out[i, cols_g[c]] += sum_k A_g[k, i] * D_g[k, c]; one block per group
__global__ void k_lmm_post(const DevGroup* __restrict__ groups, const double* __restrict__ A, int q, int nCols,
                           double* __restrict__ out, int skipFast) {
  const DevGroup& g = groups[blockIdx.x];
  if (g.type == GT_UNC || (skipFast && g.inFast)) return;
  const double* Ag = A + g.valOff * q;
  for (int e = threadIdx.x; e < q * g.gCols; e += blockDim.x) {
    const int i = e / g.gCols, c = e - i * g.gCols;
    double s = 0;
    for (int k = 0; k < g.nVals; k++) s += Ag[(size_t)k * q + i] * g.dict[(size_t)k * g.gCols + c];
    atomicAdd(&out[(size_t)i * nCols + g.cols[c]], s);
  }
}

// uncompressed group: out[i, cols[c]] += sum_r Yt[i, r] * dense[r, c]. A thread owns one column c (threads along
// the columns read a dense row contiguously) and one of `ry` row phases; the block covers a chunk of rows.
__global__ void k_lmm_unc(DevGroup g, int nRows, int rowsPerChunk, const double* __restrict__ Yt, int q, int nCols,
                          double* __restrict__ out) {
  extern __shared__ double red[];  // [ry][gCols]
  const int ra = blockIdx.x * rowsPerChunk, rb = min(nRows, ra + rowsPerChunk);
  const int gc = g.gCols;
  const int cx = threadIdx.x % gc, ry = threadIdx.x / gc, nry = blockDim.x / gc;
  for (int i = 0; i < q; i++) {
    double s = 0;
    if (ry < nry)
      for (int r = ra + ry; r < rb; r += nry) s += Yt[(size_t)i * nRows + r] * g.dense[(size_t)r * gc + cx];
    if (ry < nry) red[ry * gc + cx] = s;
    __syncthreads();
    if (ry == 0) {
      for (int k = 1; k < nry; k++) s += red[k * gc + cx];
      atomicAdd(&out[(size_t)i * nCols + g.cols[cx]], s);
    }
    __syncthreads();
  }
}

__global__ void k_lmm_unc_wide(DevGroup g, int nRows, int rowsPerChunk, const double* __restrict__ Yt, int q, int nCols,
                               double* __restrict__ out) {
  const int ra = blockIdx.x * rowsPerChunk, rb = min(nRows, ra + rowsPerChunk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nWarps = blockDim.x >> 5;
  // more columns than a block has threads: each warp owns output cells (i, c) round robin; lanes stride over rows
  for (int e = warp; e < q * g.gCols; e += nWarps) {
    const int i = e / g.gCols, c = e - i * g.gCols;
    double s = 0;
    for (int r = ra + lane; r < rb; r += 32) s += Yt[(size_t)i * nRows + r] * g.dense[(size_t)r * g.gCols + c];
    for (int d = 16; d; d >>= 1) s += __shfl_down_sync(0xffffffffu, s, d);
    if (lane == 0) atomicAdd(&out[(size_t)i * nCols + g.cols[c]], s);
  }
}

__global__ void k_row_sums(const double* __restrict__ Yt, int nRows, int q, double* __restrict__ sums) {
  const int i = blockIdx.y;
  double s = 0;
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r < nRows; r += (int64_t)gridDim.x * blockDim.x)
    s += Yt[(size_t)i * nRows + r];
  for (int d = 16; d; d >>= 1) s += __shfl_down_sync(0xffffffffu, s, d);
  if ((threadIdx.x & 31) == 0) atomicAdd(&sums[i], s);
}
__global__ void k_lmm_const(const double* __restrict__ sums, const double* __restrict__ constV, int q, int nCols,
                            double* __restrict__ out) {
  const int64_t n = (int64_t)q * nCols;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x)
    out[e] += sums[e / nCols] * constV[e % nCols];
}

// Pre-aggregation of the SDC / RLE groups for one left row from the row-major work lists: A[table row] += the left
// values of the rows an item covers. A CTA walks 1024-row blocks (left values staged in shared memory, with their
// sums per 64-row window); the block's items are read coalesced, a thread per item (an item names its step or window
// inside the block), and added to a table in shared memory that goes to A once per CTA. (The per-group form walks
// every offset stream and, for RLE, reads the whole left row once per group.) Like the general left product this
// combines partial sums with atomics.
constexpr int LL_THREADS = 256;
__global__ void __launch_bounds__(LL_THREADS)
k_lmm_lists(const SpItem* __restrict__ stepItems, const uint32_t* __restrict__ stepPtr, int64_t nStepPtr,
            const SpItem* __restrict__ winItems, const uint32_t* __restrict__ winPtr, int64_t nWinPtr, int nRows,
            const double* __restrict__ y, int nVals, double* __restrict__ A) {
  extern __shared__ __align__(16) double llsm[];
  constexpr int NSTEP = SKIP_ROWS / G3_STEP, NWIN = SKIP_ROWS / G3_WIN;
  double* ys = llsm;                        // [SKIP_ROWS]
  double* ywin = llsm + SKIP_ROWS;          // [NWIN]
  double* hist = llsm + SKIP_ROWS + NWIN;   // [nVals]
  const int tid = threadIdx.x;
  for (int i = tid; i < nVals; i += LL_THREADS) hist[i] = 0.0;
  const int nBlocks = (nRows + SKIP_ROWS - 1) / SKIP_ROWS;
  for (int b = blockIdx.x; b < nBlocks; b += gridDim.x) {
    __syncthreads();  // the previous block's readers of ys are done (and hist is cleared before the first block)
    const int r0 = b * SKIP_ROWS;
    for (int i = tid; i < SKIP_ROWS; i += LL_THREADS) ys[i] = r0 + i < nRows ? y[r0 + i] : 0.0;
    __syncthreads();
    if (tid < NWIN) {
      double sum = 0.0;
      for (int i = 0; i < G3_WIN; i++) sum += ys[tid * G3_WIN + i];
      ywin[tid] = sum;
    }
    __syncthreads();
    const int64_t w0 = (int64_t)b * NWIN, s0 = (int64_t)b * NSTEP;
    const uint32_t wa = winPtr[min(w0, nWinPtr - 1)], wb = winPtr[min(w0 + NWIN, nWinPtr - 1)];
    for (uint32_t i = wa + tid; i < wb; i += LL_THREADS) {
      const SpItem e = winItems[i];
      atomicAdd(&hist[e.prow], ywin[(e.rows >> 16) & (NWIN - 1)]);
    }
    const uint32_t sa = stepPtr[min(s0, nStepPtr - 1)], sb = stepPtr[min(s0 + NSTEP, nStepPtr - 1)];
    for (uint32_t i = sa + tid; i < sb; i += LL_THREADS) {
      const SpItem e = stepItems[i];
      const int ra = e.rows & 0xFF, rb = (e.rows >> 8) & 0xFF;
      const double* yr = ys + ((e.rows >> 16) & (NSTEP - 1)) * G3_STEP;
      double sum = 0.0;
      for (int r = ra; r < rb; r++) sum += yr[r];
      atomicAdd(&hist[e.prow], sum);
    }
  }
  __syncthreads();
  for (int i = tid; i < nVals; i += LL_THREADS) {
    const double v = hist[i];
    if (v != 0.0) atomicAdd(&A[i], v);
  }
}

int64_t launch_lmm(Matrix* m, const double* dYt, int q, double* dOut, cudaStream_t s, bool afterFast) {
  if (q == 0 || m->nCols == 0) return CLA_OK;
  if (!afterFast) CLA_CUDA(cudaMemsetAsync(dOut, 0, sizeof(double) * (size_t)q * m->nCols, s));
  if (m->nRows == 0) return CLA_OK;
  int64_t rc;
  const size_t aBytes = (size_t)std::max<int64_t>(m->totalVals, 1) * q * sizeof(double);
  const size_t sOff = (aBytes + 255) & ~(size_t)255;
  if ((rc = ensure_scratch(m, sOff + (size_t)q * sizeof(double))) < 0) return rc;
  double* A = (double*)m->scratch;
  double* sums = (double*)((char*)m->scratch + sOff);
  CLA_CUDA(cudaMemsetAsync(A, 0, sOff + (size_t)q * sizeof(double), s));
  if (m->nDev > 0) {
    const int target = std::max(1, (8 * m->smCount) / std::max(1, m->nDev));
    int rowsPerChunk = (int)(((int64_t)m->nRows + target - 1) / target);
    rowsPerChunk = std::max(SKIP_ROWS * 4, ((rowsPerChunk + SKIP_ROWS - 1) / SKIP_ROWS) * SKIP_ROWS);
    const int chunks = (m->nRows + rowsPerChunk - 1) / rowsPerChunk;
    dim3 grid(chunks, m->nDev, (q + LMM_QT - 1) / LMM_QT);
    // one left row on a tall matrix with SDC / RLE groups: those come from the row-major work lists
    bool lists = false;
    const size_t llSmem = (size_t)(SKIP_ROWS + SKIP_ROWS / G3_WIN + std::max<int64_t>(m->totalVals, 1)) * sizeof(double);
    if (q == 1 && m->nRows >= 4 * SKIP_ROWS && llSmem <= 160 * 1024) {
      if ((rc = ensure_sparse_list(m)) < 0) return rc;
      if (m->nSparse > 0) {
        if ((rc = ensure_sparse_lists(m, s)) < 0) return rc;
        lists = m->spListsOk && m->dStepPtr != nullptr;
      }
    }
    prof_begin(m, s);
    k_lmm_preagg<<<grid, LMM_THREADS, 0, s>>>(m->dGroups, m->nRows, rowsPerChunk, dYt, q, A, afterFast ? 1 : 0, lists ? 1 : 0);
    if (lists) {
      static bool llAttr[64] = {};
      if (!llAttr[m->device & 63]) {
        CLA_CUDA(cudaFuncSetAttribute(k_lmm_lists, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        llAttr[m->device & 63] = true;
      }
      const int nBlocks = (m->nRows + SKIP_ROWS - 1) / SKIP_ROWS;
      k_lmm_lists<<<std::min(nBlocks, 2 * m->smCount), LL_THREADS, llSmem, s>>>(
          (const SpItem*)m->dStepItems, m->dStepPtr, m->nStepPtr, (const SpItem*)m->dWinItems, m->dWinPtr, m->nWinPtr, m->nRows,
          dYt, (int)m->totalVals, A);
      m->stats.kernel_launches++;
    }
    prof_end(m, s);
    k_lmm_post<<<m->nDev, 128, 0, s>>>(m->dGroups, A, q, m->nCols, dOut, afterFast ? 1 : 0);
    m->stats.kernel_launches += 2;
    for (auto& g : m->groups)
      if (g.type == GT_UNC) {
        const int rpc = std::max(2048, (int)(((int64_t)m->nRows + 8 * m->smCount - 1) / (8 * m->smCount)));
        if (g.gCols <= 512) {
          const int threads = std::max(g.gCols, (512 / g.gCols) * g.gCols);  // whole multiples of the column count
          k_lmm_unc<<<(m->nRows + rpc - 1) / rpc, threads, (size_t)threads * sizeof(double), s>>>(g, m->nRows, rpc, dYt, q,
                                                                                              m->nCols, dOut);
        } else
          k_lmm_unc_wide<<<(m->nRows + rpc - 1) / rpc, 256, 0, s>>>(g, m->nRows, rpc, dYt, q, m->nCols, dOut);
        m->stats.kernel_launches++;
      }
  }
  if (m->hasConst && !afterFast) {
    dim3 grid(grid_for(m->nRows, 256, 4 * m->smCount), q);
    k_row_sums<<<grid, 256, 0, s>>>(dYt, m->nRows, q, sums);
    k_lmm_const<<<grid_for((int64_t)q * m->nCols, 256), 256, 0, s>>>(sums, m->dConstV, q, m->nCols, dOut);
    m->stats.kernel_launches += 2;
  }
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

// out += rowSums(Yt) (x) constV into a caller-provided vector of q sums
int64_t launch_lmm_const_with(Matrix* m, const double* dYt, int q, double* dOut, double* sums, cudaStream_t s) {
  if (!m->hasConst || q == 0 || m->nRows == 0) return CLA_OK;
  CLA_CUDA(cudaMemsetAsync(sums, 0, (size_t)q * sizeof(double), s));
  dim3 grid(grid_for(m->nRows, 256, 4 * m->smCount), q);
  k_row_sums<<<grid, 256, 0, s>>>(dYt, m->nRows, q, sums);
  k_lmm_const<<<grid_for((int64_t)q * m->nCols, 256), 256, 0, s>>>(sums, m->dConstV, q, m->nCols, dOut);
  m->stats.kernel_launches += 2;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

// out += rowSums(Yt) (x) constV, for callers that computed the group part themselves
int64_t launch_lmm_const(Matrix* m, const double* dYt, int q, double* dOut, cudaStream_t s) {
  if (!m->hasConst || q == 0 || m->nRows == 0) return CLA_OK;
  int64_t rc;
  if ((rc = ensure_small(m, (size_t)q * sizeof(double) + 256)) < 0) return rc;
  return launch_lmm_const_with(m, dYt, q, dOut, (double*)m->small_, s);
}

}  // namespace cla
