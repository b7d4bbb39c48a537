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
#include <climits>

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
// Second generation of the same kernel. Differences:
//  * a CTA owns a block of 1024 rows (the granularity of the skip indexes) and walks it as eight 128-row tiles,
//    so the decode state of every sparse group survives from tile to tile: one lane per SDC group keeps
//    (next listed row, its element index, stream position), one lane per RLE group keeps its current run;
//  * the lanes do not add anything themselves: they push work items {first row, last row, table row} into one
//    queue per warp (a warp owns 16 rows of the tile), and each warp then applies its own queue to its own rows
//    with plain read-modify-writes (no atomics on doubles), eight items in flight at a time;
//  * runs that cover a whole tile go to a base queue that every warp folds into two registers per lane;
//  * dense-operand columns come from a flat descriptor array (map, dictionary column, V row).
// Limits: at most 256 SDC and 256 RLE groups (8 warps x 32 lanes); larger inputs use k_rmm_dmma.
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

constexpr int Q_CAP = 512;            // items per warp queue (a power of two: sorted in place)
constexpr int QB_CAP = 512;           // base queue
constexpr int QD_CAP = 32;            // per-warp queue of run boundaries
constexpr int GM_SUB = SKIP_ROWS / GM_TR;  // tiles per block

struct WorkItem {    // read as one little-endian 64-bit key, the table row is the most significant part
  uint16_t ra, rb;   // rows [ra, rb) of the tile
  uint32_t prow;     // row of the table arena P
};
struct DeltaItem {   // rows [row, end) of the tile (inside one warp's 16-row slice) hold table row P[prow] of an RLE group
  int16_t row;
  int16_t end;
  uint32_t prow;
};
static_assert(sizeof(WorkItem) == 8 && sizeof(DeltaItem) == 8, "queue items are sorted as 64-bit keys");

// Queue slots are handed out in arrival order, which depends on warp timing; the queues are sorted by table row
// before they are applied (a group's table rows lie behind those of every earlier group, and one group never has
// two items on the same output row), so every output row receives its groups' terms in list order.
// A full queue drops the item: the count keeps growing and the tile then takes sparse_rows_in_order instead.
__device__ __forceinline__ void push_item(WorkItem* q, int* qn, int w, int ra, int rb, uint32_t prow) {
  const int slot = atomicAdd(&qn[w], 1);
  if (slot < Q_CAP) {
    WorkItem it;
    it.ra = (uint16_t)ra;
    it.rb = (uint16_t)rb;
    it.prow = prow;
    q[w * Q_CAP + slot] = it;
  }
}

// Bitonic sort of n 64-bit keys in shared memory by one warp; the array must have room for the next power of two.
__device__ __forceinline__ void warp_sort_u64(unsigned long long* a, int n) {
  const int lane = threadIdx.x & 31;
  int np = 1;
  while (np < n) np <<= 1;
  for (int i = n + lane; i < np; i += 32) a[i] = ~0ull;
  __syncwarp();
  for (int k = 2; k <= np; k <<= 1)
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = lane; t < (np >> 1); t += 32) {
        const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));  // lower index of the t-th pair at distance j
        const int l = i | j;
        const unsigned long long x = a[i], y = a[l];
        const bool up = (i & k) == 0;
        if ((x > y) == up) {
          a[i] = y;
          a[l] = x;
        }
      }
      __syncwarp();
    }
}
__device__ __forceinline__ void warp_sort_u32(uint32_t* a, int n) {
  const int lane = threadIdx.x & 31;
  int np = 1;
  while (np < n) np <<= 1;
  for (int i = n + lane; i < np; i += 32) a[i] = ~0u;
  __syncwarp();
  for (int k = 2; k <= np; k <<= 1)
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = lane; t < (np >> 1); t += 32) {
        const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
        const int l = i | j;
        const uint32_t x = a[i], y = a[l];
        const bool up = (i & k) == 0;
        if ((x > y) == up) {
          a[i] = y;
          a[l] = x;
        }
      }
      __syncwarp();
    }
}

template <bool QUAD>  // QUAD: the quad-column decode is compiled in (it costs registers the other stages then spill)
__global__ void __launch_bounds__(GM_THREADS, 2)
k_rmm_dmma2(const DevGroup* __restrict__ groups, const DenseDesc* __restrict__ dd, int nDense,
            const int32_t* __restrict__ sdcIdx, int nSdc, const int32_t* __restrict__ rleIdx, int nRle, int nRows,
            const double* __restrict__ V, int vCols, const double* __restrict__ P, const double* __restrict__ constRow,
            double* __restrict__ out) {
  extern __shared__ __align__(16) double sm[];
  double* As = sm;                      // [GM_TR][GM_LDAR] row-major stage of the dense operand
  double* Bs = sm + GM_TR * GM_LDAR;    // [GM_KC][GM_LDB]
  double* Cs = sm;                      // [GM_TR][GM_LDC] (aliases the stage)
  WorkItem* q = (WorkItem*)(sm + GM_TR * GM_LDC);      // [8][Q_CAP]
  uint32_t* qb = (uint32_t*)(q + 8 * Q_CAP);           // [QB_CAP] table rows of tile-covering runs
  DeltaItem* qd = (DeltaItem*)(qb + QB_CAP);           // [8][QD_CAP] run boundaries per warp
  int* qn = (int*)(qd + 8 * QD_CAP);                   // [8] queue lengths, [8] base queue, [9..16] boundary queues
  double* basep = (double*)(qn + 32);                  // [4][GM_TN] partial base vectors
  double* basev = basep + 4 * GM_TN;                   // [GM_TN] base vector of the tile
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int blk0 = blockIdx.x * SKIP_ROWS;
  const int j0 = blockIdx.y * GM_TN, vc = min(GM_TN, vCols - j0);
  const int am = lane >> 2, ak = lane & 3;
  const bool sparse = (nSdc + nRle) > 0;

  // ---- per-lane decode state for the whole block ----
  const int sgi = warp * 32 + lane;
  const bool hasS = sgi < nSdc, hasR = sgi < nRle;
  int sRow = INT_MAX, sElem = 0;
  int64_t sPos = 0;
  int64_t rRun = 0;
  DevGroup gs, gr;  // copies of this lane's groups (registers / local)
  if (hasS) {
    gs = groups[sdcIdx[sgi]];
    if (gs.nOff > 0) {
      if (gs.offType == CLA_OFF_BYTE || gs.offType == CLA_OFF_CHAR) {
        const SdcSkip sk = gs.skip[blockIdx.x];
        if (sk.elem < gs.nOff) {
          sRow = sk.row;
          sElem = sk.elem;
          sPos = sk.pos;
        }
      } else {  // OffsetSingle / OffsetTwo
        if (gs.first >= blk0) sRow = gs.first;
        else if (gs.offType == CLA_OFF_TWO && gs.last >= blk0) {
          sRow = gs.last;
          sElem = 1;
        }
      }
    }
  }
  if (hasR) {
    gr = groups[rleIdx[sgi]];
    rRun = gr.runSkip[blockIdx.x];
  }

  for (int sub = 0; sub < GM_SUB; sub++) {
    const int r0 = blk0 + sub * GM_TR;
    if (r0 >= nRows) break;
    const int r1 = min(nRows, r0 + GM_TR);
    double c[2][8][2];
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
      for (int nt = 0; nt < 8; nt++) c[mt][nt][0] = c[mt][nt][1] = 0.0;

    for (int k0 = 0; k0 < nDense; k0 += GM_KC) {
      const int rbase = warp * 16;
      if (QUAD && dd[k0].pad && r0 + GM_TR <= nRows) {
        // stage, all 32 columns single-column byte-map groups: a load instruction covers 8 rows x 4 adjacent
        // columns (lane = 4 * row + column). The four dictionaries of such a quad lie next to each other in the
        // packed copy, so a gather touches one or two cache lines where a lane-per-column gather touches 32 (the
        // L1 tag stage, one line per cycle, was the limit of this loop); the stores hit 16 distinct banks.
        const int kk = lane & 3, r8 = lane >> 2;
        const int rowA = r0 + rbase + r8;
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const uint8_t* mp[4];
          const double* sp[4];
#pragma unroll
          for (int g4 = 0; g4 < 4; g4++) {
            const int col = k0 + (half * 4 + g4) * 4 + kk;
            mp[g4] = nullptr;
            sp[g4] = nullptr;
            if (col < nDense) {
              mp[g4] = (const uint8_t*)dd[col].map;
              sp[g4] = dd[col].src;
            }
          }
          uint32_t id[4][2];
#pragma unroll
          for (int g4 = 0; g4 < 4; g4++)
#pragma unroll
            for (int h = 0; h < 2; h++) id[g4][h] = mp[g4] ? (uint32_t)__ldg(mp[g4] + rowA + 8 * h) : 0u;
          double vv[4][2];
#pragma unroll
          for (int g4 = 0; g4 < 4; g4++)
#pragma unroll
            for (int h = 0; h < 2; h++) vv[g4][h] = sp[g4] ? sp[g4][id[g4][h]] : 0.0;
#pragma unroll
          for (int g4 = 0; g4 < 4; g4++)
#pragma unroll
            for (int h = 0; h < 2; h++) As[(rbase + r8 + 8 * h) * GM_LDAR + (half * 4 + g4) * 4 + kk] = vv[g4][h];
        }
      } else {  // stage: warp = 16 rows of the tile, lane = one of the 32 dense columns. A dense-map column costs its lane
         // one 128-bit map load (16 ids) and 16 dictionary reads; an uncompressed column is read row by row, the
         // warp covering 32 consecutive values of a dense row. A warp-wide store is one row of the stage.
        const int kc = k0 + lane;
        double v[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = 0.0;
        if (kc < nDense) {
          const DenseDesc d = dd[kc];
          const int row0 = r0 + rbase;
          if (d.mapType < 0) {
#pragma unroll
            for (int i = 0; i < 16; i++)
              if (row0 + i < nRows) v[i] = d.src[(size_t)(row0 + i) * d.gCols];
          } else if ((d.mapType == CLA_MAP_UBYTE || d.mapType == CLA_MAP_BYTE) && row0 + 16 <= nRows) {
            const uint4 w = __ldg((const uint4*)((const uint8_t*)d.map + row0));  // row0 is a multiple of 16
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = d.src[(size_t)((ww[i >> 2] >> (8 * (i & 3))) & 0xFF) * d.gCols];
          } else {
#pragma unroll
            for (int i = 0; i < 16; i++)
              if (row0 + i < nRows) v[i] = d.src[(size_t)map_get(d.mapType, d.map, d.mapHi, row0 + i) * d.gCols];
          }
        }
#pragma unroll
        for (int i = 0; i < 16; i++) As[(rbase + i) * GM_LDAR + lane] = v[i];
      }
      {
        for (int e = tid; e < GM_KC * GM_TN; e += GM_THREADS) {
          const int kk = e >> 6, n = e & 63;
          double x = 0.0;
          if (k0 + kk < nDense && n < vc) x = V[(size_t)dd[k0 + kk].vrow * vCols + j0 + n];
          Bs[kk * GM_LDB + n] = x;
        }
      }
      __syncthreads();
#pragma unroll
      for (int ks = 0; ks < GM_KC; ks += 4) {
        double a[2];
#pragma unroll
        for (int mt = 0; mt < 2; mt++) a[mt] = As[(warp * 16 + mt * 8 + am) * GM_LDAR + ks + ak];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
          const double b = Bs[(ks + ak) * GM_LDB + nt * 8 + am];
#pragma unroll
          for (int mt = 0; mt < 2; mt++) dmma884(c[mt][nt][0], c[mt][nt][1], a[mt], b);
        }
      }
      __syncthreads();
    }

    if (!sparse) {  // straight from the fragments
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
      continue;
    }
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
      for (int nt = 0; nt < 8; nt++)
#pragma unroll
        for (int u = 0; u < 2; u++)
          Cs[(warp * 16 + mt * 8 + (lane >> 2)) * GM_LDC + nt * 8 + (lane & 3) * 2 + u] = c[mt][nt][u];
    if (tid < 17) qn[tid] = 0;
    __syncthreads();

    // ---- decode: every lane advances its groups through [r0, r1) and queues the work ----
    if (hasS) {
      const int maxV = gs.offType == CLA_OFF_BYTE ? 255 : 65535;
      while (sRow < r1) {
        if (sRow >= r0) {
          const int id = gs.single ? 0 : map_get(gs.mapType, gs.map, gs.mapHi, sElem);
          const int rl = sRow - r0;
          push_item(q, qn, rl >> 4, rl, rl + 1, (uint32_t)(gs.valOff + id));
        }
        if (sElem + 1 >= gs.nOff) {
          sRow = INT_MAX;
          break;
        }
        if (gs.offType == CLA_OFF_BYTE) {
          const uint8_t* dp = (const uint8_t*)gs.offData;
          int d = dp[sPos++];
          while (d == 0) {
            sRow += maxV;
            d = dp[sPos++];
          }
          sRow += d;
        } else if (gs.offType == CLA_OFF_CHAR) {
          const uint16_t* dp = (const uint16_t*)gs.offData;
          int d = dp[sPos++];
          while (d == 0) {
            sRow += maxV;
            d = dp[sPos++];
          }
          sRow += d;
        } else
          sRow = gs.last;  // OffsetTwo
        sElem++;
      }
    }
    if (hasR) {
      while (rRun < gr.nRuns) {
        const RleRun run = gr.runs[rRun];
        if (run.start >= r1) break;
        const int end = run.start + (int)run.len;
        const int a = max(run.start, r0), b = min(end, r1);
        if (a < b) {
          const uint32_t prow = (uint32_t)(gr.valOff + run.k);
          if (a == r0 && b == r0 + GM_TR) {
            const int slot = atomicAdd(&qn[8], 1);
            if (slot < QB_CAP) qb[slot] = prow;
            else
              for (int w = 0; w < 8; w++) push_item(q, qn, w, w * 16, w * 16 + 16, prow);
          } else {
            // a run that starts or ends inside the tile: every warp whose 16 rows it touches gets the piece of
            // the run that lies in its slice
            for (int w = (a - r0) >> 4; w <= (b - 1 - r0) >> 4; w++) {
              const int aw = max(a - r0, w * 16), bw = min(b - r0, w * 16 + 16);
              const int slot = atomicAdd(&qn[9 + w], 1);
              if (slot < QD_CAP) qd[w * QD_CAP + slot] = DeltaItem{(int16_t)aw, (int16_t)bw, prow};
              else
                push_item(q, qn, w, aw, bw, prow);
            }
          }
        }
        if (end <= r1) rRun++;
        else break;
      }
    }
    __syncthreads();

    // ---- fix the summation order: sort every queue by table row. A tile with an overflowed work queue drops its
    //      queues and takes the slow in-order walk below instead ----
    bool ovf = false;
#pragma unroll
    for (int w = 0; w < 8; w++) ovf |= qn[w] > Q_CAP;
    if (!ovf) {
      warp_sort_u64((unsigned long long*)(q + warp * Q_CAP), qn[warp]);
      warp_sort_u64((unsigned long long*)(qd + warp * QD_CAP), min(qn[9 + warp], QD_CAP));
      if (warp == 0) warp_sort_u32(qb, min(qn[8], QB_CAP));
    }
    __syncthreads();

    // ---- base vector: constV * V plus the table rows of all runs that cover the whole tile. Thread = (one of four
    //      item slices, column): every thread's loads are independent, so the whole sum costs one or two latencies ----
    {
      const int n = tid & 63, sl = tid >> 6;
      const int nbq = ovf ? 0 : min(qn[8], QB_CAP);
      double sacc = 0.0;
      if (n < vc)
        for (int i = sl; i < nbq; i += 4) sacc += P[(size_t)qb[i] * vCols + j0 + n];
      basep[sl * GM_TN + n] = sacc;
      __syncthreads();
      if (tid < GM_TN)
        basev[tid] = basep[tid] + basep[GM_TN + tid] + basep[2 * GM_TN + tid] + basep[3 * GM_TN + tid] +
                     ((constRow && tid < vc) ? constRow[j0 + tid] : 0.0);
      __syncthreads();
    }
    // ---- apply: warp w owns rows [16 w, 16 w + 16); lane owns the adjacent columns 2 lane and 2 lane + 1 ----
    {
      const int n0 = 2 * lane;
      const bool c0ok = n0 < vc, c1ok = n0 + 1 < vc;
      const bool vec2 = ((vCols | j0) & 1) == 0 && c1ok;  // table rows start 16-byte aligned and both columns exist
      auto ldp = [&](uint32_t prow) -> double2 {              // two adjacent values of a table row
        const double* p = P + (size_t)prow * vCols + j0 + n0;
        if (vec2) return *(const double2*)p;
        return make_double2(c0ok ? p[0] : 0.0, c1ok ? p[1] : 0.0);
      };
      const double2 bsum = make_double2(c0ok ? basev[n0] : 0.0, c1ok ? basev[n0 + 1] : 0.0);
      if (ovf) {
        sparse_rows_in_order(groups, nSdc, sdcIdx, P, vCols, j0, vc, Cs, r0, r1, blockIdx.x);
        sparse_rows_in_order(groups, nRle, rleIdx, P, vCols, j0, vc, Cs, r0, r1, blockIdx.x);
      }
      const int nq = ovf ? 0 : qn[warp];
      const WorkItem* myq = q + warp * Q_CAP;
      for (int i0 = 0; i0 < nq; i0 += 8) {
        double2 t[8];
        WorkItem it[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
          it[i] = myq[min(i0 + i, nq - 1)];
          t[i] = i0 + i < nq ? ldp(it[i].prow) : make_double2(0.0, 0.0);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
          if (i0 + i < nq)
            for (int r = it[i].ra; r < it[i].rb; r++) {
              double2* cp = (double2*)&Cs[r * GM_LDC + n0];
              double2 cv = *cp;
              cv.x += t[i].x;
              cv.y += t[i].y;
              *cp = cv;
            }
        }
      }
      // run pieces: eight at a time, their table rows are fetched first; then every row of the slice adds the
      // table rows of the pieces that cover it. (Walking the slice with a running sum, +P at a start and -P at an
      // end, is cheaper but leaves rounding residue of earlier, possibly much larger, values in later rows; the
      // reference adds a row's own values and nothing else.)
      const int nd = ovf ? 0 : min(qn[9 + warp], QD_CAP);
      const DeltaItem* myd = qd + warp * QD_CAP;
      for (int i0 = 0; i0 < nd; i0 += 8) {
        double2 t[8];
        int da[8], db[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const DeltaItem d = myd[min(i0 + i, nd - 1)];
          da[i] = i0 + i < nd ? d.row : 0;
          db[i] = i0 + i < nd ? d.end : 0;
          t[i] = i0 + i < nd ? ldp(d.prow) : make_double2(0.0, 0.0);
        }
        for (int r = warp * 16; r < warp * 16 + 16; r++) {
          double2 add = make_double2(0.0, 0.0);
          bool any = false;
#pragma unroll
          for (int i = 0; i < 8; i++)
            if (da[i] <= r && r < db[i]) {
              add.x += t[i].x;
              add.y += t[i].y;
              any = true;
            }
          if (any) {
            double2* cp = (double2*)&Cs[r * GM_LDC + n0];
            double2 cv = *cp;
            cv.x += add.x;
            cv.y += add.y;
            *cp = cv;
          }
        }
      }
      for (int r = warp * 16; r < warp * 16 + 16; r++) {
        if (r0 + r >= r1) break;
        const double2 cv = *(const double2*)&Cs[r * GM_LDC + n0];
        if (c0ok) out[(size_t)(r0 + r) * vCols + j0 + n0] = cv.x + bsum.x;
        if (c1ok) out[(size_t)(r0 + r) * vCols + j0 + n0 + 1] = cv.y + bsum.y;
      }
    }
    __syncthreads();  // the stage of the next tile overwrites Cs
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
  // pad of a stage's first column: 1 if the stage takes the quad-column decode: all its columns single-column
  // byte-map groups, and deep dictionaries (measured: 256 values 4.3 -> 3.2 ms on 2M x 200 x 16, but with 4 values
  // the extra byte loads and descriptor reads cost more than the saved cache-line lookups, 1.33 -> 1.59 ms per
  // 1M x 200 x 64)
  for (size_t k0 = 0; k0 < dd.size(); k0 += GM_KC) {
    bool all = true;
    int64_t vals = 0;
    const size_t k1 = std::min(dd.size(), k0 + GM_KC);
    for (size_t k = k0; k < k1; k++) {
      all &= (dd[k].mapType == CLA_MAP_UBYTE || dd[k].mapType == CLA_MAP_BYTE) && dd[k].gCols == 1;
      vals += m->groups[dc[k].group].nVals;
    }
    dd[k0].pad = (all && vals >= 64 * (int64_t)(k1 - k0)) ? 1 : 0;
    m->denseQuad |= dd[k0].pad != 0;
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
  const size_t smem2 = (size_t)GM_TR * GM_LDC * sizeof(double) + 8 * Q_CAP * sizeof(WorkItem) + QB_CAP * 4 +
                       8 * QD_CAP * sizeof(DeltaItem) + 32 * 4 + 5 * GM_TN * sizeof(double);
  static bool attrSet[64] = {};  // per device: function attributes belong to the device's context
  bool& attr = attrSet[m->device & 63];
  if (!attr) {
    CLA_CUDA(cudaFuncSetAttribute(k_rmm_dmma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CLA_CUDA(cudaFuncSetAttribute(k_rmm_dmma2<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
    CLA_CUDA(cudaFuncSetAttribute(k_rmm_dmma2<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
    attr = true;
  }
  prof_begin(m, s);
  if (m->nSdcGroups <= 256 && m->nRleGroups <= 256 && m->totalVals < (1ll << 32)) {
    dim3 grid((m->nRows + SKIP_ROWS - 1) / SKIP_ROWS, (vCols + GM_TN - 1) / GM_TN);
    auto kern = m->denseQuad ? k_rmm_dmma2<true> : k_rmm_dmma2<false>;
    kern<<<grid, GM_THREADS, smem2, s>>>(m->dGroups, (const DenseDesc*)m->dDenseDesc, m->nDenseCols,
                                               (const int32_t*)m->dSdcIdx, m->nSdcGroups, (const int32_t*)m->dRleIdx,
                                               m->nRleGroups, m->nRows, dV, vCols, P, constRow, dOut);
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
