// Products of two compressed operands on their dictionaries:
//   t(A) %*% B for two compressed blocks over the same rows (CLALibLeftMultBy.leftMultByMatrixTransposed with a
//   compressed left operand, lib/CLALibLeftMultBy.java:100-112,170-284; per pair of groups
//   APreAgg.leftMultByAColGroup / preAggregateThatIndexStructure, colgroup/APreAgg.java:70-117,211-232) and
//   t(X) %*% X on the dictionaries (lib/CLALibTSMM.java:135-154; self term AColGroupCompressed.tsmm,
//   colgroup/AColGroupCompressed.java:226-241, pair term APreAgg.tsmmAColGroup, colgroup/APreAgg.java:153-180).
//
// With X = X' + 1 c^T (c = constants, X' = the zero-default dense-map groups):
//   t(A) B = sum over pairs (g of A, h of B) of  D_g^T C_gh D_h  +  cA (x) s'B + s'A (x) cB + n cA (x) cB,
// where C_gh[i, j] = number of rows with tuple i in g and tuple j in h (the joint scan of the two maps,
// colgroup/mapping/AMapToData.java:429-493) and s' = colSums(X') = sum_g counts_g D_g. The reference adds dictionary
// rows of h into a table indexed by the ids of g, row by row; counting first and multiplying the counts with the
// dictionaries afterwards is the same sum with fewer roundings, and the counts are integers (exact, and order
// independent: the shared-memory histograms use integer atomics).
//
// Work is one integer atomic per row and pair instead of 2 * gCols_g * gCols_h flops per row: taken when every
// group of both operands is a dense-map group, every joint table has at most PAIR_MAX_CELLS cells, and there are
// fewer pairs than half the cells of the result (co-coded operands); otherwise the callers decompress row chunks
// and multiply them on the FP64 tensor cores (cla_tsmm.cu).
#include "cla_common.cuh"
#include <algorithm>
#include <cstdlib>

namespace cla {

constexpr int PAIR_MAX_CELLS = 8192;           // joint table of a pair in shared memory (32 KB of int32)
constexpr int64_t PAIR_MAX_ARENA = 16 << 20;   // joint-table cells of all pairs (128 MB of counts)
constexpr int PAIR_THREADS = 256;

struct PairDesc {
  int32_t gl, gr;      // device group indices in the left / right operand
  int64_t off;         // first cell of the pair's joint table in the arena
};

// counts1[off1[gi] + k] += rows of the chunk with tuple k, for group gi of `groups`
__global__ void __launch_bounds__(PAIR_THREADS)
k_hist1(const DevGroup* __restrict__ groups, int nRows, int rowsPerChunk, const int64_t* __restrict__ off1,
        unsigned long long* __restrict__ counts1) {
  extern __shared__ int hist[];
  const DevGroup& g = groups[blockIdx.x];
  const int nv = g.nVals;
  for (int i = threadIdx.x; i < nv; i += PAIR_THREADS) hist[i] = 0;
  __syncthreads();
  const int ra = blockIdx.y * rowsPerChunk, rb = min(nRows, ra + rowsPerChunk);
  for (int r = ra + threadIdx.x; r < rb; r += PAIR_THREADS) atomicAdd(&hist[map_get(g.mapType, g.map, g.mapHi, r)], 1);
  __syncthreads();
  for (int i = threadIdx.x; i < nv; i += PAIR_THREADS)
    if (hist[i]) atomicAdd(&counts1[off1[blockIdx.x] + i], (unsigned long long)hist[i]);
}

// joint table of every pair: counts2[off + i * nVals_r + j] += rows of the chunk with tuple i on the left and j on the right
__global__ void __launch_bounds__(PAIR_THREADS)
k_hist2(const DevGroup* __restrict__ gL, const DevGroup* __restrict__ gR, const PairDesc* __restrict__ pairs, int nRows,
        int rowsPerChunk, unsigned long long* __restrict__ counts2) {
  extern __shared__ int hist[];
  const PairDesc pd = pairs[blockIdx.x];
  const DevGroup& a = gL[pd.gl];
  const DevGroup& b = gR[pd.gr];
  const int nvb = b.nVals, cells = a.nVals * nvb;
  for (int i = threadIdx.x; i < cells; i += PAIR_THREADS) hist[i] = 0;
  __syncthreads();
  const int ra = blockIdx.y * rowsPerChunk, rb = min(nRows, ra + rowsPerChunk);
  for (int r = ra + threadIdx.x; r < rb; r += PAIR_THREADS)
    atomicAdd(&hist[map_get(a.mapType, a.map, a.mapHi, r) * nvb + map_get(b.mapType, b.map, b.mapHi, r)], 1);
  __syncthreads();
  for (int i = threadIdx.x; i < cells; i += PAIR_THREADS)
    if (hist[i]) atomicAdd(&counts2[pd.off + i], (unsigned long long)hist[i]);
}

// out[cols_g[a], cols_h[b]] += sum_i sum_j D_g[i, a] * C[i, j] * D_h[j, b]; with `mirror` also the transposed cell
// (t(X) %*% X: the pair (g, h), g < h, fills both off-diagonal blocks with the same values)
__global__ void k_pair_apply(const DevGroup* __restrict__ gL, const DevGroup* __restrict__ gR,
                             const PairDesc* __restrict__ pairs, const unsigned long long* __restrict__ counts2, int outCols,
                             double* __restrict__ out, int mirror) {
  const PairDesc pd = pairs[blockIdx.x];
  const DevGroup& g = gL[pd.gl];
  const DevGroup& h = gR[pd.gr];
  const unsigned long long* C = counts2 + pd.off;
  for (int e = threadIdx.x; e < g.gCols * h.gCols; e += blockDim.x) {
    const int a = e / h.gCols, b = e - a * h.gCols;
    double s = 0;
    for (int i = 0; i < g.nVals; i++) {
      double t = 0;  // (C D_h)[i, b]
      for (int j = 0; j < h.nVals; j++) {
        const unsigned long long c = C[(size_t)i * h.nVals + j];
        if (c) t += (double)c * h.dict[(size_t)j * h.gCols + b];
      }
      s += g.dict[(size_t)i * g.gCols + a] * t;
    }
    atomicAdd(&out[(size_t)g.cols[a] * outCols + h.cols[b]], s);
    if (mirror) atomicAdd(&out[(size_t)h.cols[b] * outCols + g.cols[a]], s);
  }
}

// t(X) %*% X, diagonal blocks: out[cols[a], cols[b]] += sum_i counts[i] * (D[i, a] * D[i, b]) (symmetric by construction)
__global__ void k_self_apply(const DevGroup* __restrict__ groups, const int64_t* __restrict__ off1,
                             const unsigned long long* __restrict__ counts1, int outCols, double* __restrict__ out) {
  const DevGroup& g = groups[blockIdx.x];
  const unsigned long long* cnt = counts1 + off1[blockIdx.x];
  for (int e = threadIdx.x; e < g.gCols * g.gCols; e += blockDim.x) {
    const int a = e / g.gCols, b = e - a * g.gCols;
    double s = 0;
    for (int i = 0; i < g.nVals; i++) s += (double)cnt[i] * (g.dict[(size_t)i * g.gCols + a] * g.dict[(size_t)i * g.gCols + b]);
    atomicAdd(&out[(size_t)g.cols[a] * outCols + g.cols[b]], s);
  }
}

// s'[cols[a]] += sum_i counts[i] * D[i, a]
__global__ void k_colsums_from_counts(const DevGroup* __restrict__ groups, const int64_t* __restrict__ off1,
                                      const unsigned long long* __restrict__ counts1, double* __restrict__ sums) {
  const DevGroup& g = groups[blockIdx.x];
  const unsigned long long* cnt = counts1 + off1[blockIdx.x];
  for (int a = threadIdx.x; a < g.gCols; a += blockDim.x) {
    double s = 0;
    for (int i = 0; i < g.nVals; i++) s += (double)cnt[i] * g.dict[(size_t)i * g.gCols + a];
    atomicAdd(&sums[g.cols[a]], s);
  }
}

// out[a, b] += cL[a] * sR[b] + sL[a] * cR[b] + n * cL[a] * cR[b]  (null constants count as zero)
__global__ void k_pair_const(const double* __restrict__ cL, const double* __restrict__ sL, const double* __restrict__ cR,
                             const double* __restrict__ sR, double n, int aCols, int bCols, double* __restrict__ out) {
  const int64_t total = (int64_t)aCols * bCols;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int a = (int)(e / bCols), b = (int)(e - (int64_t)a * bCols);
    const double ca = cL ? cL[a] : 0.0, cb = cR ? cR[b] : 0.0;
    if (ca != 0.0 || cb != 0.0) out[e] += (ca * sR[b] + sL[a] * cb) + n * (ca * cb);  // symmetric in (a, b) when L == R
  }
}

static bool pairs_disabled() {  // tuning / test aid: CLA_NO_PAIR_PREAGG=1 forces the decompress-and-multiply path
  static const bool off = getenv("CLA_NO_PAIR_PREAGG") && atoi(getenv("CLA_NO_PAIR_PREAGG")) != 0;
  return off;
}

// Every group dense-map, joint tables small, fewer pairs than half the result cells.
bool pairs_eligible(const Matrix* L, const Matrix* R, bool self) {
  if (pairs_disabled() || L->nDev == 0 || R->nDev == 0 || L->nRows < 1) return false;
  int maxL = 0, maxR = 0;
  for (auto& g : L->groups) {
    if (g.type != GT_DDC || g.nVals < 1) return false;
    maxL = std::max(maxL, g.nVals);
  }
  for (auto& g : R->groups) {
    if (g.type != GT_DDC || g.nVals < 1) return false;
    maxR = std::max(maxR, g.nVals);
  }
  if (maxL > PAIR_MAX_CELLS || maxR > PAIR_MAX_CELLS) return false;
  int64_t nPairs = 0, cells = 0;
  for (int i = 0; i < L->nDev; i++)
    for (int j = self ? i + 1 : 0; j < R->nDev; j++) {
      const int64_t c = (int64_t)L->groups[i].nVals * R->groups[j].nVals;
      if (c > PAIR_MAX_CELLS) return false;
      cells += c;
      nPairs++;
    }
  if (cells > PAIR_MAX_ARENA) return false;
  const int64_t resultCells = (int64_t)L->nCols * R->nCols / (self ? 2 : 1);
  return nPairs * 2 <= resultCells;
}

// out [aCols x bCols] = t(L) %*% R (self: L == R, upper and lower triangle both written)
int64_t launch_pairs(Matrix* L, Matrix* R, bool self, double* dOut, cudaStream_t s) {
  const int a = L->nCols, b = R->nCols;
  CLA_CUDA(cudaMemsetAsync(dOut, 0, sizeof(double) * (size_t)a * b, s));
  // arenas in L's scratch: [counts of L's groups | counts of R's groups | joint tables | s'L | s'R | offsets | pairs]
  std::vector<int64_t> off1L(L->nDev), off1R(R->nDev);
  int64_t n1 = 0;
  for (int i = 0; i < L->nDev; i++) {
    off1L[i] = n1;
    n1 += L->groups[i].nVals;
  }
  const int64_t n1L = n1;
  if (!self)
    for (int j = 0; j < R->nDev; j++) {
      off1R[j] = n1;
      n1 += R->groups[j].nVals;
    }
  std::vector<PairDesc> pairs;
  int64_t n2 = 0;
  int maxCells = 1;
  for (int i = 0; i < L->nDev; i++)
    for (int j = self ? i + 1 : 0; j < R->nDev; j++) {
      pairs.push_back(PairDesc{i, j, n2});
      const int c = L->groups[i].nVals * R->groups[j].nVals;
      n2 += c;
      maxCells = std::max(maxCells, c);
    }
  auto al = [](size_t x) { return (x + 255) & ~(size_t)255; };
  const size_t oC1 = 0, oC2 = al((size_t)n1 * 8), oSL = oC2 + al((size_t)n2 * 8), oSR = oSL + al((size_t)a * 8),
               oOffL = oSR + al((size_t)b * 8), oOffR = oOffL + al((size_t)L->nDev * 8),
               oPairs = oOffR + al((size_t)R->nDev * 8), total = oPairs + al(pairs.size() * sizeof(PairDesc));
  int64_t rc;
  if ((rc = ensure_scratch(L, total)) < 0) return rc;
  char* base = (char*)L->scratch;
  unsigned long long* c1 = (unsigned long long*)(base + oC1);
  unsigned long long* c2 = (unsigned long long*)(base + oC2);
  double* sL = (double*)(base + oSL);
  double* sR = self ? sL : (double*)(base + oSR);
  int64_t* dOffL = (int64_t*)(base + oOffL);
  int64_t* dOffR = self ? dOffL : (int64_t*)(base + oOffR);
  PairDesc* dPairs = (PairDesc*)(base + oPairs);
  CLA_CUDA(cudaMemsetAsync(base, 0, oOffL, s));  // counts and column sums start at zero
  CLA_CUDA(cudaMemcpyAsync(dOffL, off1L.data(), off1L.size() * 8, cudaMemcpyHostToDevice, s));
  if (!self) CLA_CUDA(cudaMemcpyAsync(dOffR, off1R.data(), off1R.size() * 8, cudaMemcpyHostToDevice, s));
  if (!pairs.empty()) CLA_CUDA(cudaMemcpyAsync(dPairs, pairs.data(), pairs.size() * sizeof(PairDesc), cudaMemcpyHostToDevice, s));
  CLA_CUDA(cudaStreamSynchronize(s));  // the host vectors above go out of scope with this call

  static bool attrSet[64] = {};
  bool& attr = attrSet[L->device & 63];
  if (!attr) {
    CLA_CUDA(cudaFuncSetAttribute(k_hist1, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_MAX_CELLS * 4));
    CLA_CUDA(cudaFuncSetAttribute(k_hist2, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_MAX_CELLS * 4));
    attr = true;
  }
  const int nRows = L->nRows;
  // row chunks: enough CTAs to fill the GPU a few times over, at least 16K rows each
  auto chunking = [&](int64_t units, int* rowsPerChunk) {
    const int64_t want = std::max<int64_t>(1, (8LL * L->smCount + units - 1) / std::max<int64_t>(units, 1));
    int64_t rpc = std::max<int64_t>(16384, ((int64_t)nRows + want - 1) / want);
    *rowsPerChunk = (int)std::min<int64_t>(rpc, std::max(nRows, 1));
    return (int)(((int64_t)nRows + *rowsPerChunk - 1) / *rowsPerChunk);
  };
  int rpc1 = 0;
  int maxV = 1;
  for (auto& g : L->groups) maxV = std::max(maxV, g.nVals);
  for (auto& g : R->groups) maxV = std::max(maxV, g.nVals);
  {
    const int chunks = chunking(L->nDev, &rpc1);
    k_hist1<<<dim3(L->nDev, chunks), PAIR_THREADS, (size_t)maxV * 4, s>>>(L->dGroups, nRows, rpc1, dOffL, c1);
    L->stats.kernel_launches++;
  }
  if (!self) {
    const int chunks = chunking(R->nDev, &rpc1);
    k_hist1<<<dim3(R->nDev, chunks), PAIR_THREADS, (size_t)maxV * 4, s>>>(R->dGroups, nRows, rpc1, dOffR, c1);
    L->stats.kernel_launches++;
  }
  (void)n1L;
  if (!pairs.empty()) {
    int rpc2 = 0;
    const int chunks = chunking((int64_t)pairs.size(), &rpc2);
    prof_begin(L, s);
    k_hist2<<<dim3((unsigned)pairs.size(), chunks), PAIR_THREADS, (size_t)maxCells * 4, s>>>(L->dGroups, R->dGroups, dPairs, nRows,
                                                                                          rpc2, c2);
    prof_end(L, s);
    k_pair_apply<<<(unsigned)pairs.size(), 128, 0, s>>>(L->dGroups, R->dGroups, dPairs, c2, b, dOut, self ? 1 : 0);
    L->stats.kernel_launches += 2;
  }
  if (self) {
    k_self_apply<<<L->nDev, 128, 0, s>>>(L->dGroups, dOffL, c1, b, dOut);
    L->stats.kernel_launches++;
  }
  if (L->hasConst || R->hasConst) {
    k_colsums_from_counts<<<L->nDev, 64, 0, s>>>(L->dGroups, dOffL, c1, sL);
    if (!self) k_colsums_from_counts<<<R->nDev, 64, 0, s>>>(R->dGroups, dOffR, c1, sR);
    const int64_t cells = (int64_t)a * b;
    k_pair_const<<<(unsigned)std::max<int64_t>(1, std::min<int64_t>(1024, (cells + 255) / 256)), 256, 0, s>>>(
        L->hasConst ? L->dConstV : nullptr, sL, R->hasConst ? R->dConstV : nullptr, sR, (double)nRows, a, b, dOut);
    L->stats.kernel_launches += 3;
  }
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

}  // namespace cla
