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
#include <cub/cub.cuh>
#include <algorithm>
#include <climits>
#include <cstdlib>

namespace cla {

constexpr int GM_TR = 128;     // rows per CTA
constexpr int GM_TN = 64;      // output columns per CTA
constexpr int GM_KC = 32;      // dense columns per stage
constexpr int GM_LDA = 132;    // A^T row stride (doubles), = 4 mod 16: conflict-free fragment loads
constexpr int GM_LDAR = 36;    // row-major stage stride (second-generation kernel), = 4 mod 16
constexpr int GM_LDB = 68;     // V tile row stride, = 4 mod 16
constexpr int GM_LDC = 66;     // C tile row stride
constexpr int GM_THREADS = 256;

__device__ __forceinline__ void dmma884(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c0), "+d"(c1)
               : "d"(a), "d"(b));
}

// m16n8k8 (PTX ISA fragment layout, g = lane >> 2, t = lane & 3): a0 (g, t), a1 (g + 8, t), a2 (g, t + 4),
// a3 (g + 8, t + 4); b0 (k = t, n = g), b1 (k = t + 4, n = g); c0 (g, 2t), c1 (g, 2t + 1), c2 (g + 8, 2t), c3 (g + 8, 2t + 1)
__device__ __forceinline__ void dmma1688(double& c0, double& c1, double& c2, double& c3, double a0, double a1, double a2,
                                         double a3, double b0, double b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+d"(c0), "+d"(c1), "+d"(c2), "+d"(c3)
               : "d"(a0), "d"(a1), "d"(a2), "d"(a3), "d"(b0), "d"(b1));
}

struct DenseCol {
  int32_t group;  // device group index
  int32_t j;      // column inside the group
  int32_t col;    // matrix column (row of V)
  int32_t pad;
};

// Adds the SDC and RLE groups to a 128-row tile of partial results in shared memory, in list order and without
// atomics: warp w owns rows [16 w, 16 w + 16) of the tile and walks the groups one after the other (`list` = their
// device group indices, or null: every group of `groups`). An SDC group is decoded from the skip entry of its
// 1024-row block (32 deltas per step, warp scan); the lane that finds a listed row adds that row's table row. An
// RLE group's runs are clipped to the warp's rows; lane n adds columns n and n + 32. This is the slow, always
// available form: the second-generation kernel uses it when one of its work queues overflows.
__device__ __forceinline__ void sparse_rows_in_order(const DevGroup* __restrict__ groups, int n,
                                                     const int32_t* __restrict__ list, const double* __restrict__ P,
                                                     int vCols, int j0, int vc, double* Cs, int r0, int r1, int skipBlock) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ra = r0 + warp * 16, rb = min(r1, ra + 16);
  if (ra >= rb) return;
  for (int i = 0; i < n; i++) {
    const DevGroup& g = groups[list ? list[i] : i];
    if (g.type == GT_SDC) {
      const double* Pg = P + g.valOff * vCols + j0;
      sdc_walk_block(g, ra, rb, [&](int row, int e) {
        const int id = g.single ? 0 : map_get(g.mapType, g.map, g.mapHi, e);
        double* cr = Cs + (row - r0) * GM_LDC;
        const double* p = Pg + (size_t)id * vCols;
        for (int c = 0; c < vc; c++) cr[c] += p[c];
      });
      __syncwarp();
    } else if (g.type == GT_RLE) {
      const double* Pg = P + g.valOff * vCols + j0;
      for (int64_t ri = g.runSkip[skipBlock]; ri < g.nRuns; ri++) {
        const RleRun run = g.runs[ri];
        if (run.start >= rb) break;
        const int a = max(run.start, ra), b = min(run.start + (int)run.len, rb);
        if (a >= b) continue;
        const double* p = Pg + (size_t)run.k * vCols;
        const double p0 = lane < vc ? p[lane] : 0.0, p1 = lane + 32 < vc ? p[lane + 32] : 0.0;
        for (int r = a; r < b; r++) {
          if (lane < vc) Cs[(r - r0) * GM_LDC + lane] += p0;
          if (lane + 32 < vc) Cs[(r - r0) * GM_LDC + lane + 32] += p1;
        }
      }
      __syncwarp();
    }
  }
}

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
  // ---- sparse groups: warp w owns rows [16 w, 16 w + 16) of the tile and adds every group in list order ----
  sparse_rows_in_order(groups, nGroups, nullptr, P, vCols, j0, vc, Cs, r0, r1, blockIdx.x * GM_TR / SKIP_ROWS);
  __syncthreads();
  for (int e = tid; e < GM_TR * GM_TN; e += GM_THREADS) {
    const int r = e >> 6, n = e & 63;
    if (r0 + r < r1 && n < vc) out[(size_t)(r0 + r) * vCols + j0 + n] = Cs[r * GM_LDC + n] + base[n];
  }
}

// --------------------------------------------------------------------------------------------------
// Second generation. The CTAs are persistent (one per SM) and hold the rows of V that belong to the dense-operand
// columns in shared memory for their whole life, so nothing in the main loop needs a CTA-wide barrier: every warp
// works on its own 512-row units, 16 rows at a time, independently of the others. For its 16 rows a warp
//   1. decodes 32 dense-operand columns at a time (lane = column: one 128-bit map load and 16 dictionary reads,
//      or 16 values of an uncompressed column) into its private stage and multiplies it with the resident rows of
//      V by DMMA m8n8k4, accumulators in registers; the map word of the stage after next and the dictionary reads
//      of the next stage are in flight meanwhile, and while one warp waits the other seven keep the tensor pipe busy;
//   2. moves the accumulators to its private result tile and adds the SDC and RLE groups from their
//      pre-aggregated tables P_g = D_g * V[cols_g, :], walking the work lists built once per matrix by
//      build_sparse_lists (below): per 16-row step the pieces {first row, end row, table row} of every listed SDC
//      row and of every RLE run that starts or ends inside a 64-row window, sorted by group, so that each output
//      row receives its terms in the groups' list order without any queue or atomic; and per 64-row window the
//      table rows of the RLE runs that cover the window entirely, which are summed once per window into a vector
//      held in registers. Sixteen table rows are in flight at a time;
//   3. adds constV * V and writes the 16 rows out, 512 contiguous bytes per row.
// Dense-operand columns beyond what fits shared memory next to the warps' tiles are handled by further launches
// that add to the result.
// --------------------------------------------------------------------------------------------------
struct DenseDesc {
  const void* map;     // map (dense-map groups) or null
  const void* mapHi;
  const double* src;   // dictionary + j, or dense block + j
  int32_t mapType;     // -1: uncompressed
  int32_t gCols;
  int32_t vrow;        // row of V (= matrix column)
  int32_t pad;
};


// NT = 8-column tiles per CTA (8: 64 output columns, two per lane in the sparse phase; 4: 32 columns, one per lane),
// WARPS = warps per CTA, IB = table rows in flight per warp in the sparse phase. With eight warps the SM issued 0.9
// instructions per clock (two warps per scheduler, every instruction waiting out the latency of the one before) and
// neither the tensor pipe nor the L1 data pipe was busy; sixteen warps must fit 128 registers and spill; twelve is
// the measured optimum for the 64-column tile. The per-warp buffers are sized so that sixteen fit next to V.
template <int NT, int WARPS>
struct G3 {
  static constexpr int TN = NT * 8;
  static constexpr int LDB = TN + 4;    // = 4 mod 16: conflict-free fragment loads
  static constexpr int LDC = TN + 2;    // row stride of a warp's result tile (8 rows at a time)
  static constexpr int WBUF = 16 * GM_LDAR > G3_STEP * LDC ? 16 * GM_LDAR : G3_STEP * LDC;  // doubles per warp: stage [16][GM_LDAR], then the tile
  static constexpr int THREADS = WARPS * 32;
  static constexpr int CPL = TN / 32;   // output columns per lane in the sparse phase
  static constexpr int KMAX = ((227 * 1024 - 1024 - WARPS * WBUF * 8) / (LDB * 8)) / GM_KC * GM_KC;  // resident rows of V
};

template <int NT, int WARPS, int IB>
__global__ void __launch_bounds__(WARPS * 32, 1)
k_rmm_dmma3(const DenseDesc* __restrict__ dd, int nDense, const SpItem* __restrict__ stepItems,
            const uint32_t* __restrict__ stepPtr, const SpItem* __restrict__ winItems,
            const uint32_t* __restrict__ winPtr, int nRows, const double* __restrict__ V, int vCols,
            const double* __restrict__ P, const double* __restrict__ constRow, double* __restrict__ out, int accumulate) {
  typedef G3<NT, WARPS> C;
  constexpr int TN = C::TN, LDB = C::LDB, LDC = C::LDC, CPL = C::CPL;
  extern __shared__ __align__(16) double sm[];
  const int nSt = (nDense + GM_KC - 1) / GM_KC;  // stages of 32 dense-operand columns
  const int kPad = nSt * GM_KC;
  double* Vs = sm;                                   // [kPad][LDB]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  double* W = sm + (size_t)kPad * LDB + warp * C::WBUF;  // this warp's stage / result tile
  const int j0 = blockIdx.y * TN, vc = min(TN, vCols - j0);
  for (int e = tid; e < kPad * TN; e += C::THREADS) {
    const int kc = e / TN, n = e - kc * TN;
    Vs[kc * LDB + n] = (kc < nDense && n < vc) ? V[(size_t)dd[kc].vrow * vCols + j0 + n] : 0.0;
  }
  __syncthreads();
  const int am = lane >> 2, ak = lane & 3;
  const int n0 = CPL * lane;  // this lane's output column(s) in the result tile
  const bool c0ok = n0 < vc, c1ok = CPL == 2 && n0 + 1 < vc;
  const bool vec2 = CPL == 2 && ((vCols | j0) & 1) == 0 && c1ok;  // rows of P and out start 16-byte aligned, both columns exist
  const char* Pb = (const char*)(P + j0 + n0);   // this lane's columns of table row 0
  const uint32_t rowBytes = (uint32_t)vCols * 8u;  // the launcher checks that the whole table stays below 4 GB
  char* Wb = (char*)(W + n0);                     // this lane's columns of row 0 of the result tile
  const double2 cst = make_double2((constRow && c0ok) ? constRow[j0 + n0] : 0.0, (constRow && c1ok) ? constRow[j0 + n0 + 1] : 0.0);

  // Decode of one stage for 16 rows, split so that the map word of stage t + 2 and the dictionary reads of stage
  // t + 1 are in flight while stage t multiplies: map word first (byte maps, full 16 rows) ...
  auto stage_map = [&](int r0, int r1, int k0) -> uint4 {
    const int kc = k0 + lane;
    if (kc < nDense && r0 + 16 <= r1) {
      const int mt = dd[kc].mapType;
      if (mt == CLA_MAP_UBYTE || mt == CLA_MAP_BYTE) return __ldg((const uint4*)((const uint8_t*)dd[kc].map + r0));
    }
    return make_uint4(0, 0, 0, 0);
  };
  // ... then the values
  auto stage_values = [&](int r0, int r1, int k0, const uint4& w, double (&v)[16]) {
    const int kc = k0 + lane;
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = 0.0;
    if (kc >= nDense) return;
    const DenseDesc d = dd[kc];
    if (d.mapType < 0) {
#pragma unroll
      for (int i = 0; i < 16; i++)
        if (r0 + i < r1) v[i] = d.src[(size_t)(r0 + i) * d.gCols];
    } else if ((d.mapType == CLA_MAP_UBYTE || d.mapType == CLA_MAP_BYTE) && r0 + 16 <= r1) {
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 16; i++) v[i] = d.src[(size_t)((ww[i >> 2] >> (8 * (i & 3))) & 0xFF) * d.gCols];
    } else {
#pragma unroll
      for (int i = 0; i < 16; i++)
        if (r0 + i < r1) v[i] = d.src[(size_t)map_get(d.mapType, d.map, d.mapHi, r0 + i) * d.gCols];
    }
  };

  const int nUnits = (nRows + G3_UNIT - 1) / G3_UNIT;
  for (int unit = blockIdx.x * WARPS + warp; unit < nUnits; unit += gridDim.x * WARPS) {
    const int U0 = unit * G3_UNIT, U1 = min(nRows, U0 + G3_UNIT);
    // list bounds of the unit's 64 steps and 8 windows: lane l holds the starts of steps l and 32 + l (window l); the
    // end of the last one is the start of the next unit's first
    uint32_t sp0 = 0, sp1 = 0, spEnd = 0, wp = 0, wpEnd = 0;
    if (stepPtr) {
      sp0 = stepPtr[unit * (G3_UNIT / G3_STEP) + lane];
      sp1 = stepPtr[unit * (G3_UNIT / G3_STEP) + 32 + lane];
      spEnd = stepPtr[(unit + 1) * (G3_UNIT / G3_STEP)];
      wp = winPtr[unit * (G3_UNIT / G3_WIN) + (lane & 7)];
      wpEnd = winPtr[(unit + 1) * (G3_UNIT / G3_WIN)];
    }
    const int nSub = (U1 - U0 + 15) / 16;
    uint4 wq = nSt > 0 ? stage_map(U0, U1, 0) : make_uint4(0, 0, 0, 0);  // the map word is fetched one stage ahead
    double baseWin[CPL];
#pragma unroll
    for (int q = 0; q < CPL; q++) baseWin[q] = 0.0;
    for (int sub = 0; sub < nSub; sub++) {
      const int r0 = U0 + sub * 16, r1 = min(U1, r0 + 16);
      double c[2][NT][2];
      if (accumulate) {
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int u = 0; u < 2; u++) {
              const int row = r0 + mt * 8 + am, n = nt * 8 + ak * 2 + u;
              c[mt][nt][u] = (row < r1 && n < vc) ? out[(size_t)row * vCols + j0 + n] : 0.0;
            }
      } else {
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
          for (int nt = 0; nt < NT; nt++) c[mt][nt][0] = c[mt][nt][1] = 0.0;
      }
      for (int st = 0; st < nSt; st++) {
        const int k0 = st * GM_KC;
        {
          double v[16];
          stage_values(r0, r1, k0, wq, v);
          __syncwarp();  // the previous stage's fragment loads (or the previous step's stores) are done
#pragma unroll
          for (int i = 0; i < 16; i++) W[i * GM_LDAR + lane] = v[i];
        }
        {  // map word of the next stage
          const bool lastSt = st + 1 == nSt;
          const int nr0 = lastSt ? r0 + 16 : r0, nk0 = lastSt ? 0 : k0 + GM_KC;
          if (nr0 < U1) wq = stage_map(nr0, U1 < nr0 + 16 ? U1 : nr0 + 16, nk0);
        }
        __syncwarp();
        // m16n8k8: the 16 staged rows are one A tile, so a quarter of the tensor instructions of the m8n8k4 form for
        // the same fragment loads (both shapes run at the same rate; the kernel is short of issue slots, not of math)
#pragma unroll
        for (int ks = 0; ks < GM_KC; ks += 8) {
          const double a0 = W[am * GM_LDAR + ks + ak], a1 = W[(8 + am) * GM_LDAR + ks + ak];
          const double a2 = W[am * GM_LDAR + ks + 4 + ak], a3 = W[(8 + am) * GM_LDAR + ks + 4 + ak];
#pragma unroll
          for (int nt = 0; nt < NT; nt++) {
            const double b0 = Vs[(k0 + ks + ak) * LDB + nt * 8 + am], b1 = Vs[(k0 + ks + 4 + ak) * LDB + nt * 8 + am];
            dmma1688(c[0][nt][0], c[0][nt][1], c[1][nt][0], c[1][nt][1], a0, a1, a2, a3, b0, b1);
          }
        }
      }
      // ---- the two 8-row halves: accumulators -> result tile, sparse groups from the work lists, constants, store.
      //      One copy of this code (no unrolling over the halves or the two lists): with sixteen warps at different
      //      places of the kernel, instruction fetch was the largest stall of the fully unrolled form. ----
#pragma unroll 1
      for (int h = 0; h < 2; h++) {
        const int h0 = r0 + h * G3_STEP, h1 = min(r1, h0 + G3_STEP);
        if (h0 >= h1) break;
        __syncwarp();
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
          *(double2*)&W[am * LDC + nt * 8 + ak * 2] =
              make_double2(h ? c[1][nt][0] : c[0][nt][0], h ? c[1][nt][1] : c[0][nt][1]);
        __syncwarp();
        double base[CPL];
#pragma unroll
        for (int q = 0; q < CPL; q++) base[q] = 0.0;
        if (stepPtr) {
          const bool whole = h1 - h0 == G3_STEP;
          const int step = sub * 2 + h;
          const bool newWin = (step & 7) == 0;  // a new 64-row window: first the runs that cover it entirely
          if (newWin) {
#pragma unroll
            for (int q = 0; q < CPL; q++) baseWin[q] = 0.0;
          }
          const int w = step >> 3;
          const uint32_t q0 = __shfl_sync(0xffffffffu, wp, w), q1n = __shfl_sync(0xffffffffu, wp, (w + 1) & 7);
          const uint32_t pa = __shfl_sync(0xffffffffu, step < 32 ? sp0 : sp1, step & 31);
          const uint32_t pbn = __shfl_sync(0xffffffffu, step + 1 < 32 ? sp0 : sp1, (step + 1) & 31);
#pragma unroll 1
          for (int pass = newWin ? 0 : 1; pass < 2; pass++) {
            const bool toWin = pass == 0;
            const SpItem* __restrict__ items = toWin ? winItems : stepItems;
            const uint32_t p0 = toWin ? q0 : pa, p1 = toWin ? (w == 7 ? wpEnd : q1n) : (step == 63 ? spEnd : pbn);
            // items [p0, p1): 32 per coalesced load; every lane turns its own item into the byte offset of the table
            // row and a word {offset of the first row in the tile, number of rows, "add to the base vector"} once,
            // so that the serial part per item is two shuffles, one load and one read-modify-write. IB table
            // rows are in flight at a time; items are applied in list order.
#pragma unroll 1
            for (uint32_t i0 = p0; i0 < p1; i0 += 32) {
              const int cnt = (int)min(32u, p1 - i0);
              uint32_t offP = 0, wrd = 0;
              if (lane < cnt) {
                const SpItem e = items[i0 + lane];
                const uint32_t ra = e.rows & 0xFF, nr = ((e.rows >> 8) & 0xFF) - ra;
                offP = e.prow * rowBytes;
                wrd = (ra * (uint32_t)(LDC * 8)) | (nr << 16) | ((toWin || (whole && nr == G3_STEP)) ? 0x80000000u : 0u);
              }
#pragma unroll 1
              for (int b0 = 0; b0 < cnt; b0 += IB) {
                double2 t[IB];
                uint32_t rw[IB];
                const int nb = min(IB, cnt - b0);
#pragma unroll
                for (int j = 0; j < IB; j++) {
                  const uint32_t po = __shfl_sync(0xffffffffu, offP, (b0 + j) & 31);
                  rw[j] = __shfl_sync(0xffffffffu, wrd, (b0 + j) & 31);
                  if (j < nb) {
                    const char* pp = Pb + po;
                    if (vec2) t[j] = *(const double2*)pp;
                    else t[j] = make_double2(c0ok ? ((const double*)pp)[0] : 0.0, c1ok ? ((const double*)pp)[1] : 0.0);
                  }
                }
#pragma unroll
                for (int j = 0; j < IB; j++) {
                  if (j < nb) {
                    if (rw[j] & 0x80000000u) {  // covers the whole step (or window): one add to a vector in registers
                      if (toWin) {
                        baseWin[0] += t[j].x;
                        if (CPL == 2) baseWin[CPL - 1] += t[j].y;
                      } else {
                        base[0] += t[j].x;
                        if (CPL == 2) base[CPL - 1] += t[j].y;
                      }
                    } else {
                      char* cp = Wb + (rw[j] & 0xFFFFu);
                      int nr = (int)((rw[j] >> 16) & 0xFF);
                      do {
                        if (CPL == 2) {
                          double2 cv = *(double2*)cp;
                          cv.x += t[j].x;
                          cv.y += t[j].y;
                          *(double2*)cp = cv;
                        } else
                          *(double*)cp += t[j].x;
                        cp += LDC * 8;
                      } while (--nr > 0);
                    }
                  }
                }
              }
            }
          }
        }
        __syncwarp();
#pragma unroll 1
        for (int r = 0; r < h1 - h0; r++) {
          double* o = out + (size_t)(h0 + r) * vCols + j0 + n0;
          if (CPL == 2) {
            const double2 cv = *(const double2*)&W[r * LDC + n0];
            const double x = ((cv.x + base[0]) + baseWin[0]) + cst.x, y = ((cv.y + base[CPL - 1]) + baseWin[CPL - 1]) + cst.y;
            if (vec2) *(double2*)o = make_double2(x, y);
            else {
              if (c0ok) o[0] = x;
              if (c1ok) o[1] = y;
            }
          } else if (c0ok)
            o[0] = ((W[r * LDC + n0] + base[0]) + baseWin[0]) + cst.x;
        }
      }
    }
  }
}

// --------------------------------------------------------------------------------------------------
// Work lists of the sparse phase, built once per matrix (first wide right product): the SDC and RLE groups turned
// from per-group index structures into per-row-range lists. A warp per (group, 1024-row block) decodes the block
// (offset stream from its skip entry, runs from the merged run list) and emits
//   * per 8-row step: {rows [ra, rb) of the step, table row} for every listed SDC row and for every piece of an RLE
//     run that lies in a 64-row window the run does not cover entirely;
//   * per 64-row window: {table row} for every RLE run that covers the window entirely.
// Both lists are sorted by (step or window, table row); table rows grow with the group index, so within a step the
// items are in the groups' list order. The ptr arrays hold the start of every step / window (padded to whole units).
// --------------------------------------------------------------------------------------------------
__global__ void k_sparse_emit(const DevGroup* __restrict__ groups, const int32_t* __restrict__ sparseIdx, int nSparse,
                              int nRows, unsigned long long* __restrict__ stepKeys, uint32_t* __restrict__ stepVals,
                              unsigned long long* __restrict__ winKeys, unsigned long long* __restrict__ counters) {
  const int lane = threadIdx.x & 31;
  const int64_t warpId = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int nBlocks = (nRows + SKIP_ROWS - 1) / SKIP_ROWS;
  const int gi = (int)(warpId / nBlocks), blk = (int)(warpId % nBlocks);
  if (gi >= nSparse) return;
  const DevGroup& g = groups[sparseIdx[gi]];
  const int b0 = blk * SKIP_ROWS, b1 = min(nRows, b0 + SKIP_ROWS);
  auto emit_step = [&](int row0, int row1, uint32_t prow) {  // rows [row0, row1) inside one step
    const unsigned long long slot = atomicAdd(&counters[0], 1ull);
    if (stepKeys) {
      stepKeys[slot] = ((unsigned long long)(row0 / G3_STEP) << 32) | prow;
      stepVals[slot] = (uint32_t)(row0 % G3_STEP) | ((uint32_t)(row1 - row0 / G3_STEP * G3_STEP) << 8) |
                       ((uint32_t)((row0 / G3_STEP) % (SKIP_ROWS / G3_STEP)) << 16);  // + the step's place in its 1024-row block
    }
  };
  if (g.type == GT_SDC) {
    sdc_walk_block(g, b0, b1, [&](int row, int e) {
      const int id = g.single ? 0 : map_get(g.mapType, g.map, g.mapHi, e);
      emit_step(row, row + 1, (uint32_t)(g.valOff + id));
    });
  } else if (g.type == GT_RLE) {
    for (int64_t ri = g.runSkip[blk] + lane; ri < g.nRuns; ri += 32) {
      const RleRun R = g.runs[ri];
      if (R.start >= b1) break;
      const int a = max(R.start, b0), b = min(R.start + (int)R.len, b1);
      const uint32_t prow = (uint32_t)(g.valOff + R.k);
      for (int w0 = a & ~(G3_WIN - 1); w0 < b; w0 += G3_WIN) {
        const int wa = max(a, w0), wb = min(b, w0 + G3_WIN);
        if (wa >= wb) continue;
        if (wb - wa == G3_WIN) {
          const unsigned long long slot = atomicAdd(&counters[1], 1ull);
          if (winKeys) winKeys[slot] = ((unsigned long long)(w0 / G3_WIN) << 32) | prow;
        } else {
          for (int s0 = wa / G3_STEP * G3_STEP; s0 < wb; s0 += G3_STEP) {
            const int sa = max(wa, s0), sb = min(wb, s0 + G3_STEP);
            if (sa < sb) emit_step(sa, sb, prow);
          }
        }
      }
    }
  }
}
// items[i] = {table row, rows}; ptr[u] = first item whose step / window is >= u
__global__ void k_sparse_pack(const unsigned long long* __restrict__ keys, const uint32_t* __restrict__ vals, int64_t n,
                              SpItem* __restrict__ items) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    SpItem it;
    it.prow = (uint32_t)keys[i];
    // window items carry the window's place in its 1024-row block where step items carry the step's
    it.rows = vals ? vals[i] : (uint32_t)((keys[i] >> 32) % (SKIP_ROWS / G3_WIN)) << 16;
    items[i] = it;
  }
}
__global__ void k_sparse_ptr(const unsigned long long* __restrict__ keys, int64_t n, uint32_t* __restrict__ ptr, int64_t nPtr) {
  for (int64_t u = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; u < nPtr; u += (int64_t)gridDim.x * blockDim.x) {
    int64_t lo = 0, hi = n;  // first key with (key >> 32) >= u
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if ((int64_t)(keys[mid] >> 32) < u) lo = mid + 1;
      else hi = mid;
    }
    ptr[u] = (uint32_t)lo;
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

// Builds (once per handle) the lists the kernels walk: dense-operand columns, SDC groups, RLE groups.
static int64_t ensure_dense_cols(Matrix* m) {
  if (m->denseColsBuilt) return CLA_OK;
  std::vector<DenseCol> dc;
  std::vector<DenseDesc> dd;
  std::vector<int32_t> sdc, rle;
  // The staging loop reads the dictionaries of 32 different columns with one gather. Registered one by one they
  // each start a cache line of their own, so such a gather touches 32 lines; a packed copy of all dense-map
  // dictionaries brings small ones (4 values = 32 bytes) four to a line.
  size_t packDoubles = 0;
  for (int gi = 0; gi < m->nDev; gi++)
    if (m->groups[gi].type == GT_DDC) packDoubles += (size_t)m->groups[gi].nVals * m->groups[gi].gCols;
  double* packed = nullptr;
  if (packDoubles) {
    cudaError_t e = cudaMalloc((void**)&packed, packDoubles * sizeof(double));
    if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc packed dictionaries: ") + cudaGetErrorString(e));
    m->allocs.push_back(packed);
  }
  size_t packAt = 0;
  for (int gi = 0; gi < m->nDev; gi++) {
    const DevGroup& g = m->groups[gi];
    if (g.type == GT_SDC) sdc.push_back(gi);
    if (g.type == GT_RLE) rle.push_back(gi);
    if (g.type != GT_DDC && g.type != GT_UNC) continue;
    const double* dictAt = g.dict;
    if (g.type == GT_DDC) {
      const size_t n = (size_t)g.nVals * g.gCols;
      CLA_CUDA(cudaMemcpy(packed + packAt, g.dict, n * sizeof(double), cudaMemcpyDeviceToDevice));
      dictAt = packed + packAt;
      packAt += n;
    }
    std::vector<int32_t> cols(g.gCols);
    CLA_CUDA(cudaMemcpy(cols.data(), g.cols, cols.size() * 4, cudaMemcpyDeviceToHost));
    for (int j = 0; j < g.gCols; j++) {
      dc.push_back(DenseCol{gi, j, cols[j], 0});
      DenseDesc d;
      d.map = g.type == GT_UNC ? nullptr : g.map;
      d.mapHi = g.mapHi;
      d.src = (g.type == GT_UNC ? g.dense : dictAt) + j;
      d.mapType = g.type == GT_UNC ? -1 : g.mapType;
      d.gCols = g.gCols;
      d.vrow = cols[j];
      d.pad = 0;
      dd.push_back(d);
    }
  }
  auto up = [&](const void* src, size_t bytes, void** dst) -> int64_t {
    *dst = nullptr;
    if (!bytes) return CLA_OK;
    cudaError_t e = cudaMalloc(dst, bytes);
    if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc column lists: ") + cudaGetErrorString(e));
    m->allocs.push_back(*dst);
    CLA_CUDA(cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice));
    return CLA_OK;
  };
  int64_t rc;
  if ((rc = up(dc.data(), dc.size() * sizeof(DenseCol), &m->dDenseCols)) < 0) return rc;
  if ((rc = up(dd.data(), dd.size() * sizeof(DenseDesc), &m->dDenseDesc)) < 0) return rc;
  if ((rc = up(sdc.data(), sdc.size() * 4, &m->dSdcIdx)) < 0) return rc;
  if ((rc = up(rle.data(), rle.size() * 4, &m->dRleIdx)) < 0) return rc;
  m->nDenseCols = (int)dc.size();
  m->nSdcGroups = (int)sdc.size();
  m->nRleGroups = (int)rle.size();
  m->denseColsBuilt = true;
  return CLA_OK;
}

// Builds the work lists (see k_sparse_emit). Returns CLA_OK with m->spListsOk = false when the lists would not fit
// 32-bit positions or device memory; the caller then takes the first-generation kernel.
int64_t ensure_sparse_lists(Matrix* m, cudaStream_t s) {
  if (m->spListsTried) return CLA_OK;
  m->spListsTried = true;
  int64_t rc;
  if ((rc = ensure_sparse_list(m)) < 0) return rc;
  if (m->nSparse == 0 || m->nRows == 0) {
    m->spListsOk = true;  // nothing to add: the kernel is told so by null lists
    return CLA_OK;
  }
  if (m->totalVals >= (1ll << 32)) return CLA_OK;
  const int nBlocks = (m->nRows + SKIP_ROWS - 1) / SKIP_ROWS;
  const int64_t warps = (int64_t)m->nSparse * nBlocks;
  const unsigned grid = (unsigned)((warps * 32 + 255) / 256);
  unsigned long long* dCnt = nullptr;
  CLA_CUDA(cudaMalloc((void**)&dCnt, 2 * sizeof(unsigned long long)));
  auto fail_free = [&](std::vector<void*> ps, int64_t code, const std::string& msg) {
    for (void* p : ps)
      if (p) cudaFree(p);
    cudaFree(dCnt);
    return code == CLA_OK ? CLA_OK : fail(code, msg);
  };
  CLA_CUDA(cudaMemsetAsync(dCnt, 0, 2 * sizeof(unsigned long long), s));
  k_sparse_emit<<<grid, 256, 0, s>>>(m->dGroups, m->dSparseIdx, m->nSparse, m->nRows, nullptr, nullptr, nullptr, dCnt);  // count
  unsigned long long cnt[2] = {0, 0};
  CLA_CUDA(cudaMemcpyAsync(cnt, dCnt, sizeof(cnt), cudaMemcpyDeviceToHost, s));
  CLA_CUDA(cudaStreamSynchronize(s));
  const int64_t nStep = (int64_t)cnt[0], nWin = (int64_t)cnt[1];
  if (nStep >= (1ll << 31) || nWin >= (1ll << 31)) return fail_free({}, CLA_OK, "");
  const int nUnits = (m->nRows + G3_UNIT - 1) / G3_UNIT;
  const int64_t nStepPtr = (int64_t)nUnits * (G3_UNIT / G3_STEP) + 1, nWinPtr = (int64_t)nUnits * (G3_UNIT / G3_WIN) + 1;
  // sort buffers (freed below), then the final lists
  unsigned long long *k0 = nullptr, *k1 = nullptr, *wk0 = nullptr, *wk1 = nullptr;
  uint32_t *v0 = nullptr, *v1 = nullptr;
  void* tmp = nullptr;
  auto A = [&](void** p, size_t bytes) { return cudaMalloc(p, std::max<size_t>(bytes, 16)) == cudaSuccess; };
  if (!A((void**)&k0, nStep * 8) || !A((void**)&k1, nStep * 8) || !A((void**)&v0, nStep * 4) || !A((void**)&v1, nStep * 4) ||
      !A((void**)&wk0, nWin * 8) || !A((void**)&wk1, nWin * 8)) {
    cudaGetLastError();
    return fail_free({k0, k1, v0, v1, wk0, wk1}, CLA_OK, "");
  }
  CLA_CUDA(cudaMemsetAsync(dCnt, 0, 2 * sizeof(unsigned long long), s));
  k_sparse_emit<<<grid, 256, 0, s>>>(m->dGroups, m->dSparseIdx, m->nSparse, m->nRows, k0, v0, wk0, dCnt);
  size_t tb1 = 0, tb2 = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, tb1, k0, k1, v0, v1, (int)nStep, 0, 64, s);
  cub::DeviceRadixSort::SortKeys(nullptr, tb2, wk0, wk1, (int)nWin, 0, 64, s);
  if (!A(&tmp, std::max(tb1, tb2))) {
    cudaGetLastError();
    return fail_free({k0, k1, v0, v1, wk0, wk1}, CLA_OK, "");
  }
  if (nStep) cub::DeviceRadixSort::SortPairs(tmp, tb1, k0, k1, v0, v1, (int)nStep, 0, 64, s);
  if (nWin) cub::DeviceRadixSort::SortKeys(tmp, tb2, wk0, wk1, (int)nWin, 0, 64, s);
  void *stepItems = nullptr, *winItems = nullptr, *stepPtr = nullptr, *winPtr = nullptr;
  if (!A(&stepItems, nStep * sizeof(SpItem)) || !A(&winItems, nWin * sizeof(SpItem)) || !A(&stepPtr, nStepPtr * 4) ||
      !A(&winPtr, nWinPtr * 4)) {
    cudaGetLastError();
    return fail_free({k0, k1, v0, v1, wk0, wk1, tmp, stepItems, winItems, stepPtr, winPtr}, CLA_OK, "");
  }
  const unsigned long long* sk = nStep ? k1 : k0;
  const unsigned long long* wk = nWin ? wk1 : wk0;
  k_sparse_pack<<<1184, 256, 0, s>>>(sk, nStep ? v1 : v0, nStep, (SpItem*)stepItems);
  k_sparse_pack<<<1184, 256, 0, s>>>(wk, nullptr, nWin, (SpItem*)winItems);
  k_sparse_ptr<<<(unsigned)((nStepPtr + 255) / 256), 256, 0, s>>>(sk, nStep, (uint32_t*)stepPtr, nStepPtr);
  k_sparse_ptr<<<(unsigned)((nWinPtr + 255) / 256), 256, 0, s>>>(wk, nWin, (uint32_t*)winPtr, nWinPtr);
  CLA_CUDA(cudaStreamSynchronize(s));
  CLA_CUDA(cudaGetLastError());
  for (void* p : {(void*)k0, (void*)k1, (void*)v0, (void*)v1, (void*)wk0, (void*)wk1, tmp, (void*)dCnt}) cudaFree(p);
  for (void* p : {stepItems, winItems, stepPtr, winPtr}) m->allocs.push_back(p);
  m->dStepItems = stepItems;
  m->dWinItems = winItems;
  m->dStepPtr = (uint32_t*)stepPtr;
  m->dWinPtr = (uint32_t*)winPtr;
  m->nStepPtr = nStepPtr;
  m->nWinPtr = nWinPtr;
  m->deviceBytes += (nStep + nWin) * (int64_t)sizeof(SpItem) + (nStepPtr + nWinPtr) * 4;
  m->stats.device_bytes = m->deviceBytes;
  m->spListsOk = true;
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
  if ((rc = ensure_sparse_lists(m, s)) < 0) return rc;
  static bool attrSet[64] = {};  // per device: function attributes belong to the device's context
  bool& attr = attrSet[m->device & 63];
  if (!attr) {
    CLA_CUDA(cudaFuncSetAttribute(k_rmm_dmma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CLA_CUDA(cudaFuncSetAttribute(k_rmm_dmma3<8, 12, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    CLA_CUDA(cudaFuncSetAttribute(k_rmm_dmma3<8, 16, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    CLA_CUDA(cudaFuncSetAttribute(k_rmm_dmma3<4, 16, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    attr = true;
  }
  prof_begin(m, s);
  if (m->spListsOk && (m->nSparse == 0 || (int64_t)m->totalVals * vCols * 8 < (1ll << 32))) {  // table-row offsets are 32-bit
    static const int wideEnv = getenv("CLA_RMM_WIDE_TILES") ? atoi(getenv("CLA_RMM_WIDE_TILES")) : -1;  // tuning aid
    const bool wide = wideEnv >= 0 ? wideEnv != 0 : vCols > 32;  // 64 output columns per CTA, or 32
    const int nUnits = (m->nRows + G3_UNIT - 1) / G3_UNIT;
    // 64-column tile: 12 warps of 166 registers are 9 % faster per row than 16 warps of 128 (which spill), but a warp
    // works on whole 512-row units, so below two units per warp the 16-warp CTA finishes in fewer rounds (1M rows:
    // 2.6 ms against 3.5 ms under the profiler; 4M rows: 9.8 against 8.9 ms)
    const bool w12 = wide && nUnits >= 2 * 12 * std::max(1, m->smCount / ((vCols + 63) / 64));  // CTAs along the rows
    const int TN = wide ? 64 : 32, W = w12 ? 12 : 16;
    const int kMax = wide ? (w12 ? G3<8, 12>::KMAX : G3<8, 16>::KMAX) : G3<4, 16>::KMAX;
    const int ldb = TN + 4, wbuf = wide ? (w12 ? G3<8, 12>::WBUF : G3<8, 16>::WBUF) : G3<4, 16>::WBUF;
    const int gridY = (vCols + TN - 1) / TN;
    dim3 grid((unsigned)std::max(1, std::min(std::max(1, m->smCount / gridY), (nUnits + W - 1) / W)), gridY);
    const DenseDesc* dd = (const DenseDesc*)m->dDenseDesc;
    int k0 = 0;
    do {  // dense-operand columns in slices that fit shared memory; the first launch also adds the sparse groups
      const int nk = std::min(kMax, m->nDenseCols - k0);
      const bool first = k0 == 0;
      const size_t smem3 = ((size_t)((nk + GM_KC - 1) / GM_KC * GM_KC) * ldb + (size_t)W * wbuf) * sizeof(double);
      // 64-column tile: 12 warps of up to 170 registers (no spills; 16 warps of 128 registers spilled 320 bytes) and 8
      // table rows in flight in the sparse phase. Measured on 4M rows of the mixed benchmark matrix, ms per product:
      // 8 / 10 / 12 / 14 / 16 warps 10.8 / 10.5 / 8.9 / 9.4 / 9.8; with 12 warps 2 / 4 / 8 table rows 10.0 / 9.0 / 8.9.
      auto kern = wide ? (w12 ? k_rmm_dmma3<8, 12, 8> : k_rmm_dmma3<8, 16, 4>) : k_rmm_dmma3<4, 16, 8>;
      kern<<<grid, W * 32, smem3, s>>>(dd + k0, nk, first ? (const SpItem*)m->dStepItems : nullptr,
                                       first ? m->dStepPtr : nullptr, (const SpItem*)m->dWinItems, m->dWinPtr, m->nRows, dV,
                                       vCols, P, first ? constRow : nullptr, dOut, first ? 0 : 1);
      m->stats.kernel_launches++;
      k0 += nk;
    } while (k0 < m->nDenseCols);
    m->stats.kernel_launches--;  // counted once more below
  } else {
    dim3 grid((m->nRows + GM_TR - 1) / GM_TR, (vCols + GM_TN - 1) / GM_TN);
    k_rmm_dmma<<<grid, GM_THREADS, smem, s>>>(m->dGroups, m->nDev, (const DenseCol*)m->dDenseCols, m->nDenseCols, m->nRows,
                                             dV, vCols, P, constRow, dOut, hasSparse);
  }
  prof_end(m, s);
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

}  // namespace cla
