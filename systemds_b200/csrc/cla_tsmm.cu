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
#include <cstdlib>

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

// m16n8k8: eight times the flops of m8n8k4 per instruction and, per flop, half the B-fragment bytes (a 16-row tile
// reuses each B value for twice the rows). Fragments (PTX ISA, mma.m16n8k8 .f64): a0 (g, t), a1 (g + 8, t),
// a2 (g, t + 4), a3 (g + 8, t + 4); b0 (k = t, n = g), b1 (k = t + 4, n = g); c0 (g, 2t), c1 (g, 2t + 1),
// c2 (g + 8, 2t), c3 (g + 8, 2t + 1), with g = lane >> 2, t = lane & 3.
__device__ __forceinline__ void dmma1688(double (&c)[4], double a0, double a1, double a2, double a3, double b0, double b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
               : "d"(a0), "d"(a1), "d"(a2), "d"(a3), "d"(b0), "d"(b1));
}

// Loads pinned where they are written: volatile asm is not moved across the (volatile) DMMAs, so a load issued
// before a block of DMMAs stays in flight during them instead of being sunk to its first use behind them.
__device__ __forceinline__ double ld_f64_here(const double* p) {
  double v;
  asm volatile("ld.global.nc.f64 %0, [%1];" : "=d"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_u8_here(const uint8_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_u16_here(const uint16_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// grid: (blocks of A columns x blocks of B columns, k splits). A: [rows x aCols], B: [rows x bCols], both row-major
// chunks of the same rows. C [aCols x bCols] += A^T B. A CTA owns one 64 x 64 block of C; warp w its rows 8 w .. 8 w + 8.
// 16-row stages, double buffered (static shared memory, 35 KB): the loads of the next stage are issued into registers before the DMMAs of the
// current one and stored to the other buffer after them, so one barrier per stage and no exposed load latency.
// SYRK: B is A, blockIdx.x enumerates the block pairs bi <= bj of the upper triangle, only cells on or above the
// diagonal are added (t(X) %*% X with more than 128 columns).
constexpr int GT_KT = 16;
template <bool SYRK>
__global__ void __launch_bounds__(TS_THREADS)
k_gemm_tn_dmma(const double* __restrict__ A, int aCols, const double* __restrict__ B, int bCols, int rows, int nBlkB,
               double* __restrict__ C, int rowsPerSplit) {
  __shared__ double sI[2][GT_KT * TS_LD];
  __shared__ double sJ[2][GT_KT * TS_LD];
  int bi, bj;
  if (SYRK) {  // decode the linear pair index into (bi <= bj)
    int p = blockIdx.x;
    bi = 0;
    while (p >= nBlkB - bi) {
      p -= nBlkB - bi;
      bi++;
    }
    bj = bi + p;
  } else {
    bi = blockIdx.x / nBlkB;
    bj = blockIdx.x - bi * nBlkB;
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rBeg = blockIdx.y * rowsPerSplit, rEnd = min(rows, rBeg + rowsPerSplit);
  if (rBeg >= rEnd) return;
  double c[8][2];
#pragma unroll
  for (int t = 0; t < 8; t++) c[t][0] = c[t][1] = 0.0;
  const int am = lane >> 2, ak = lane & 3;
  // this thread's cells of a stage: column cc of rows kk0, kk0 + 4, ... (GT_KT * 64 / 256 = 4 cells per operand)
  const int cc = tid & 63, kk0 = tid >> 6;
  const int ci = bi * TS_BLK + cc, cj = bj * TS_BLK + cc;
  constexpr int GT_CELLS = GT_KT * TS_BLK / TS_THREADS;
  double va[GT_CELLS], vb[GT_CELLS];
  auto load = [&](int r) {
#pragma unroll
    for (int u = 0; u < GT_CELLS; u++) {
      const int row = r + kk0 + 4 * u;
      va[u] = (row < rEnd && ci < aCols) ? ld_f64_here(A + (size_t)row * aCols + ci) : 0.0;
      vb[u] = (row < rEnd && cj < bCols) ? ld_f64_here(B + (size_t)row * bCols + cj) : 0.0;
    }
  };
  auto store = [&](int buf) {
#pragma unroll
    for (int u = 0; u < GT_CELLS; u++) {
      sI[buf][(kk0 + 4 * u) * TS_LD + cc] = va[u];
      sJ[buf][(kk0 + 4 * u) * TS_LD + cc] = vb[u];
    }
  };
  load(rBeg);
  store(0);
  __syncthreads();
  int cur = 0;
  for (int r = rBeg; r < rEnd; r += GT_KT) {
    const bool more = r + GT_KT < rEnd;
    if (more) load(r + GT_KT);
#pragma unroll
    for (int k0 = 0; k0 < GT_KT; k0 += 4) {
      const double a = sI[cur][(k0 + ak) * TS_LD + warp * 8 + am];  // A[m][k] = A[k][bi*64 + warp*8 + m]
#pragma unroll
      for (int t = 0; t < 8; t++) dmma884(c[t][0], c[t][1], a, sJ[cur][(k0 + ak) * TS_LD + t * 8 + am]);
    }
    if (more) store(cur ^ 1);
    __syncthreads();
    cur ^= 1;
  }
  const int gi = bi * TS_BLK + warp * 8 + (lane >> 2);
#pragma unroll
  for (int t = 0; t < 8; t++) {
#pragma unroll
    for (int u = 0; u < 2; u++) {
      const int gj = bj * TS_BLK + t * 8 + (lane & 3) * 2 + u;
      if (gi < aCols && gj < bCols && (!SYRK || gi <= gj) && c[t][u] != 0.0) atomicAdd(&C[(size_t)gi * bCols + gj], c[t][u]);
    }
  }
}

// --------------------------------------------------------------------------------------------------
// Up to 128 columns: one CTA holds the whole upper triangle of the result as 16x8 DMMA tiles, so nothing of the
// product is computed twice and only the triangle's tiles are computed at all. Rows are split across CTAs; each
// adds its partial triangle to the result with atomics at the end.
// FUSED: the 32-row stage is decoded straight from the maps and dictionaries (dense-map and uncompressed groups
// only), so the dense form of X never exists, not even in L2. Otherwise the stage is read from a decompressed chunk.
// --------------------------------------------------------------------------------------------------
constexpr int TT_KT = 32;             // rows per stage

// What the staging loop needs to know about one matrix column, kept in shared memory.
struct TsmmCol {
  const void* map;     // null: no dense-map / uncompressed group holds the column
  const void* mapHi;
  const double* src;   // dictionary (or the dense block) already offset to the column inside the group
  double cst;          // constant part of the column
  int32_t mapType;     // -1: uncompressed (src is the dense block + j)
  int32_t gCols;
};

// --------------------------------------------------------------------------------------------------
// 16 warps in one CTA per SM. The triangle's tiles are dealt to the warps as contiguous runs of the row-major tile
// order (TPW tiles each, so a warp's A fragment changes at most a few times), which keeps the accumulators at
// 2 * TPW registers per thread and leaves room for a two-deep register pipeline of the decode: while the DMMAs of stage s run, the dictionary gathers of stage s+2 and the map loads
// of stage s+3 are in flight; their values go to one of four shared-memory stage buffers an iteration later.
// (An earlier 8-warp version, whose decode had to finish, values in shared memory, before its DMMAs started,
// stalled 7.6 cycles per issue on those gathers; this one 0.5.)
// --------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

constexpr int T16_WARPS = 16;
constexpr int T16_THREADS = T16_WARPS * 32;
constexpr int T16_MAXC = 8;   // columns decoded per warp and stage at 128 columns

// SIMPLE (with MT = byte or char): every column is held by a dense-map group of that width, so a column needs two
// pointers (map, dictionary) instead of the full record, whose reads were 40 % of the kernel's shared-memory load
// instructions. SIMPLE = 1: single-column groups and no constant part; SIMPLE = 2: also the group width (co-coded
// columns) and the constant part of the column.
// The MMAs of one 32-row stage on 16 x 8 tiles for a warp that owns N of its TPW tile slots. N is a template
// parameter, not a predicate on each MMA: a predicated-off MMA still takes its turn in the tensor pipe.
// The fragments of k-step ks + 8 are loaded before the MMAs of k-step ks are issued.
template <int N, int TPW, int LD>
__device__ __forceinline__ void tsmm_stage_1688(const double* __restrict__ Xt, const int (&offA)[TPW], const int (&offB)[TPW],
                                                uint32_t aMask, double (&c)[TPW][4]) {
  double2 bC[N], aC0 = *(const double2*)&Xt[offA[0]], aC1 = *(const double2*)&Xt[offA[0] + 8 * LD];
#pragma unroll
  for (int sl = 0; sl < N; sl++) bC[sl] = *(const double2*)&Xt[offB[sl]];
#pragma unroll
  for (int ks = 0; ks < 32; ks += 8) {
    double2 bN[N], aN0 = make_double2(0.0, 0.0), aN1 = make_double2(0.0, 0.0);
    if (ks + 8 < 32) {
      aN0 = *(const double2*)&Xt[offA[0] + ks + 8];
      aN1 = *(const double2*)&Xt[offA[0] + 8 * LD + ks + 8];
#pragma unroll
      for (int sl = 0; sl < N; sl++) bN[sl] = *(const double2*)&Xt[offB[sl] + ks + 8];
    }
    double2 a0 = aC0, a1 = aC1;
#pragma unroll
    for (int sl = 0; sl < N; sl++) {
      if (sl > 0 && ((aMask >> sl) & 1u)) {
        a0 = *(const double2*)&Xt[offA[sl] + ks];
        a1 = *(const double2*)&Xt[offA[sl] + 8 * LD + ks];
      }
      dmma1688(c[sl], a0.x, a1.x, a0.y, a1.y, bC[sl].x, bC[sl].y);
    }
    if (ks + 8 < 32) {
      aC0 = aN0;
      aC1 = aN1;
#pragma unroll
      for (int sl = 0; sl < N; sl++) bC[sl] = bN[sl];
    }
  }
}

// The triangle is cut into 16 x 8 tiles for m16n8k8 (8 x 8 tiles on m8n8k4 needed twice the B-fragment bytes per
// flop and four times the instructions; measured 10.6 -> 10.3 ms on 20M x 100). The stage keeps its rows (the k dimension) in the
// order 0, 4, 1, 5, 2, 6, 3, 7 within every group of eight, so that the two k values a lane needs of an A or B
// fragment are adjacent: one 128-bit load per fragment half; its stride TT_LDB = 8 mod 16 makes those loads
// conflict free (a quarter-warp reads 64 contiguous bytes of two columns).
constexpr int TT_LDB = TT_KT + 8;
template <bool FUSED, int MT, int TPW, int SIMPLE>
__global__ void __launch_bounds__(T16_THREADS, 1)
k_tsmm_tri16(const DevGroup* __restrict__ groups, const int32_t* __restrict__ colSrc, const double* __restrict__ constV,
             const double* __restrict__ X, int rowBegin, int rowEnd, int nCols, double* __restrict__ C, int32_t* err) {
  extern __shared__ __align__(16) double XtAll[];  // four stages of [nColsPad][TT_LDB], the column records, four mbarriers
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int LD = TT_LDB;
  constexpr int CW = 4;                             // accumulator doubles per tile slot
  const int NT = (nCols + 7) >> 3;                  // 8-column tiles
  const int NI = (nCols + 15) >> 4;                 // tile rows (16 matrix columns each)
  const int nColsPad = NI * 16;                     // columns of the stage (zero beyond nCols)
  const int stageDoubles = nColsPad * LD;
  TsmmCol* cols = (TsmmCol*)(XtAll + 4 * stageDoubles);
  uint64_t* bars = (uint64_t*)(cols + nColsPad);
  if (tid == 0) {
    for (int b = 0; b < 4; b++) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars[b])), "r"(T16_THREADS));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (FUSED) {
    for (int cc = tid; cc < nColsPad; cc += T16_THREADS) {
      TsmmCol d;
      d.map = nullptr;
      d.mapHi = nullptr;
      d.src = nullptr;
      d.cst = (constV && cc < nCols) ? constV[cc] : 0.0;
      d.mapType = 0;
      d.gCols = 1;
      if (cc < nCols && colSrc[2 * cc] >= 0) {
        const DevGroup& g = groups[colSrc[2 * cc]];
        const int j = colSrc[2 * cc + 1];
        d.gCols = g.gCols;
        if (g.type == GT_UNC) {
          d.mapType = -1;
          d.src = g.dense + j;
          d.map = g.dense;  // non-null marker
        } else {
          d.mapType = g.mapType;
          d.map = g.mapType == CLA_MAP_ZERO ? (const void*)g.dict : g.map;
          d.mapHi = g.mapHi;
          d.src = g.dict + j;
        }
      }
      cols[cc] = d;
    }
    __syncthreads();
  }
  // SIMPLE: the two pointers per column, packed behind the mbarriers
  const void** mapArr = (const void**)(bars + 4);
  const double** srcArr = (const double**)(mapArr + nColsPad);
  double* cstArr = (double*)(srcArr + nColsPad);
  int* gcArr = (int*)(cstArr + nColsPad);
  if (SIMPLE) {
    for (int cc = tid; cc < nColsPad; cc += T16_THREADS) {
      mapArr[cc] = cols[cc].map;
      srcArr[cc] = cols[cc].src;
      cstArr[cc] = cols[cc].cst;
      gcArr[cc] = cols[cc].gCols;
    }
    __syncthreads();
  }
  // this warp's tiles: [t0, t1) of the row-major order of the upper triangle
  // tile row I holds the tiles (I, J) with J >= firstJ(I): every 8-column tile that reaches the diagonal or lies above it
  auto rowLen = [&](int I) { return NT - 2 * I; };
  auto firstJ = [&](int I) { return 2 * I; };
  const int nTiles = NI * NT - NI * (NI - 1);
  const int t0 = nTiles * warp / T16_WARPS, t1 = nTiles * (warp + 1) / T16_WARPS;
  const int am = lane >> 2, ak = lane & 3;
  // Fragment offsets of each of the TPW tile slots. A slot the warp does not own points at tile (0, 0) and its
  // accumulator is never written out: the inner loop then needs no test per slot. aMask bit sl: slot sl starts
  // a new tile row, i.e. needs a fresh A fragment (bit 0 always).
  int offA[TPW], offB[TPW];
  uint32_t aMask = 1;
  {
    int I = 0, base = 0;  // base = linear index of the first tile of row I
    while (I < NI && base + rowLen(I) <= t0) {
      base += rowLen(I);
      I++;
    }
    int J = firstJ(I) + (t0 - base);
#pragma unroll
    for (int sl = 0; sl < TPW; sl++) {
      if (t0 + sl < t1) {
        offA[sl] = (I * 16 + am) * LD + 2 * ak;
        offB[sl] = (J * 8 + am) * LD + 2 * ak;
        if (J == firstJ(I)) aMask |= 1u << sl;
        if (++J == NT) {
          I++;
          J = firstJ(I);
        }
      } else {
        offA[sl] = offB[sl] = am * LD + 2 * ak;
        aMask |= 1u << sl;
      }
    }
  }
  const int nMine = t1 - t0;
  double c[TPW][CW];
#pragma unroll
  for (int i = 0; i < TPW; i++)
#pragma unroll
    for (int u = 0; u < CW; u++) c[i][u] = 0.0;

  const int64_t nStages = ((int64_t)(rowEnd - rowBegin) + TT_KT - 1) / TT_KT;
  const int64_t sa = nStages * blockIdx.x / gridDim.x, sb = nStages * (blockIdx.x + 1) / gridDim.x;
  if (sa >= sb) return;

  // ---- decode pipeline: column warp + 16 * b of the stage, lanes along the 32 rows ----
  uint32_t ids[T16_MAXC];  // dictionary ids of the stage two ahead
  double vals[T16_MAXC];   // values of the stage one ahead
  auto load_ids = [&](int64_t st) {
    if (!FUSED) return;
    const int row = rowBegin + (int)st * TT_KT + lane;
    const bool inRange = row < rowEnd;
#pragma unroll
    for (int b = 0; b < T16_MAXC; b++) {
      const int cc = warp + T16_WARPS * b;
      ids[b] = 0;
      if (SIMPLE) {
        if (cc < nCols && inRange)
          ids[b] = MT == CLA_MAP_BYTE ? ld_u8_here((const uint8_t*)mapArr[cc] + row) : ld_u16_here((const uint16_t*)mapArr[cc] + row);
      } else if (cc < nColsPad && inRange) {
        const TsmmCol& d = cols[cc];
        if (d.map && d.mapType >= 0) {
          // the raw id only: any arithmetic on it here would wait for the load
          if (MT == CLA_MAP_BYTE) ids[b] = ld_u8_here((const uint8_t*)d.map + row);
          else if (MT == CLA_MAP_CHAR) ids[b] = ld_u16_here((const uint16_t*)d.map + row);
          else ids[b] = (uint32_t)map_get(d.mapType, d.map, d.mapHi, row);
        }
      }
    }
  };
  auto gather = [&](int64_t st) {  // issues the loads of a stage's values (uses ids for dense-map columns)
    const int row = rowBegin + (int)st * TT_KT + lane;
    const bool inRange = row < rowEnd;
#pragma unroll
    for (int b = 0; b < T16_MAXC; b++) {
      const int cc = warp + T16_WARPS * b;
      vals[b] = 0.0;
      if (SIMPLE) {
        if (cc < nCols && inRange) vals[b] = ld_f64_here(srcArr[cc] + (SIMPLE == 2 ? (size_t)ids[b] * gcArr[cc] : (size_t)ids[b]));
      } else if (cc < nColsPad && inRange) {
        // volatile asm keeps the load where it is written, ahead of the (volatile) DMMAs: left to itself the
        // compiler sinks it to its use behind them and the pipeline is gone
        if (FUSED) {
          const TsmmCol& d = cols[cc];
          if (d.map) vals[b] = ld_f64_here(d.src + (d.mapType < 0 ? (size_t)row : (size_t)ids[b]) * d.gCols);
        } else if (cc < nCols)
          vals[b] = ld_f64_here(X + (size_t)(row - rowBegin) * nCols + cc);
      }
    }
  };
  auto store = [&](int64_t st, double* Xt) {  // adds the constant part of the column (rows inside the matrix only)
    const bool inRange = rowBegin + (int)st * TT_KT + lane < rowEnd;
#pragma unroll
    for (int b = 0; b < T16_MAXC; b++) {
      const int cc = warp + T16_WARPS * b;
      if (cc < nColsPad)
        Xt[cc * LD + ((lane & ~7) | ((lane & 3) << 1) | ((lane >> 2) & 1))] =
            vals[b] + ((FUSED && inRange && SIMPLE != 1) ? (SIMPLE == 2 ? cstArr[cc] : cols[cc].cst) : 0.0);
    }
  };
  // Four stage buffers, each with an mbarrier that counts the 512 threads' "my part of this stage is stored". A warp
  // stores its part of stage s + 1 and signals, issues the loads of the stages behind it, and only then waits for
  // stage s -- which every warp finished storing a whole iteration earlier -- so the warps drift up to a stage apart
  // and their DMMA phases no longer coincide (with one __syncthreads per stage they did: the tensor pipe was 47 %
  // busy yet throttling). Buffer (s + 1) % 4 was last read by the DMMAs of stage s - 3; a warp that is about to
  // store stage s + 1 has seen stage s - 1 complete, i.e. every warp had stored it, which each did after its
  // DMMAs of stage s - 3: no barrier is needed before the store.
  auto bar_addr = [&](int b) { return smem_addr(&bars[b]); };
  auto signal = [&](int b) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_addr(b)) : "memory"); };
  auto wait_for = [&](int b, uint32_t parity) -> bool {  // bounded: gives up after 2^20 polls and reports it
    uint32_t done = 0;
    for (int it = 0; it < (1 << 20) && !done; it++)
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(done)
                   : "r"(bar_addr(b)), "r"(parity)
                   : "memory");
    return done != 0;
  };
  load_ids(sa);
  gather(sa);
  store(sa, XtAll);
  signal(0);
  if (sa + 1 < sb) {
    load_ids(sa + 1);
    gather(sa + 1);
  }
  if (sa + 2 < sb) load_ids(sa + 2);
  for (int64_t st = sa; st < sb; st++) {
    const int it = (int)(st - sa);
    if (st + 1 < sb) {  // vals holds stage st + 1 (gathered one iteration ago)
      store(st + 1, XtAll + ((it + 1) & 3) * stageDoubles);
      signal((it + 1) & 3);
    }
    if (st + 2 < sb) gather(st + 2);    // addresses from ids (loaded one iteration ago)
    if (st + 3 < sb) load_ids(st + 3);  // then the registers take the ids of the stage after that
    if (!wait_for(it & 3, (uint32_t)(it >> 2) & 1u)) {
      if (lane == 0) atomicExch(err, 7);  // stage never completed: give up, the host reports the self-check
      return;
    }
    const double* Xt = XtAll + (it & 3) * stageDoubles;
    // k-step outermost, tile slots innermost: consecutive DMMAs go to different accumulators, so none waits for
    // the one before it; no branch in the loop body (the A reload is a predicated load)
    // (the fragments of k-step ks + 4 are loaded into registers before the DMMAs of k-step ks are issued, so the
    // shared-memory latency is covered by the warp's own DMMAs rather than by the three other warps of its scheduler)
    {
      static_assert(TT_KT == 32, "tsmm_stage_1688 walks 32 rows");
      if (nMine == TPW) tsmm_stage_1688<TPW, TPW, LD>(Xt, offA, offB, aMask, c);
      else if (nMine == TPW - 1) tsmm_stage_1688<(TPW > 1 ? TPW - 1 : 1), TPW, LD>(Xt, offA, offB, aMask, c);
      else if (nMine == TPW - 2) tsmm_stage_1688<(TPW > 2 ? TPW - 2 : 1), TPW, LD>(Xt, offA, offB, aMask, c);
      else if (nMine > 0) tsmm_stage_1688<1, TPW, LD>(Xt, offA, offB, aMask, c);
    }
  }
  // ---- add the partial tiles ----
  {
    int I = 0, base = 0;
    while (I < NI && base + rowLen(I) <= t0) {
      base += rowLen(I);
      I++;
    }
    int J = firstJ(I) + (t0 - base);
#pragma unroll
    for (int sl = 0; sl < TPW; sl++) {
      if (t0 + sl < t1) {
#pragma unroll
        for (int u = 0; u < CW; u++) {
          const int gi = I * 16 + (lane >> 2) + 8 * (u >> 1);
          const int gj = J * 8 + (lane & 3) * 2 + (u & 1);
          if (gi < nCols && gj < nCols && gi <= gj && c[sl][u] != 0.0) atomicAdd(&C[(size_t)gi * nCols + gj], c[sl][u]);
        }
        if (++J == NT) {
          I++;
          J = firstJ(I);
        }
      }
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

// --------------------------------------------------------------------------------------------------
// FP64 peak probes: the denominators for the tensor-pipe and FMA-pipe fractions quoted for the kernels above.
// --------------------------------------------------------------------------------------------------
__global__ void k_peak_dmma(int iters, double* sink) {
  double c[8][2];
#pragma unroll
  for (int i = 0; i < 8; i++) c[i][0] = c[i][1] = 0.0;
  const double a = 1.0 + threadIdx.x * 1e-9, b = 1.0 - threadIdx.x * 1e-9;
  for (int it = 0; it < iters; it++) {
#pragma unroll
    for (int i = 0; i < 8; i++) dmma884(c[i][0], c[i][1], a, b);
  }
  double s = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) s += c[i][0] + c[i][1];
  if (s == 12345.678) sink[0] = s;  // keeps the loop alive
}
__global__ void k_peak_dfma(int iters, double* sink) {
  double c[16];
#pragma unroll
  for (int i = 0; i < 16; i++) c[i] = threadIdx.x * 1e-3 + i;
  const double a = 1.0000001, b = 1e-9;
  for (int it = 0; it < iters; it++) {
#pragma unroll
    for (int i = 0; i < 16; i++) c[i] = fma(c[i], a, b);
  }
  double s = 0;
#pragma unroll
  for (int i = 0; i < 16; i++) s += c[i];
  if (s == 12345.678) sink[0] = s;
}

// TFLOP/s of back-to-back DMMA m8n8k4 (512 flop per warp instruction) and of FP64 FMA, on `device`.
int64_t measure_fp64_peaks(int device, double* dmmaTflops, double* dfmaTflops) {
  CLA_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  CLA_CUDA(cudaGetDeviceProperties(&prop, device));
  double* sink = nullptr;
  CLA_CUDA(cudaMalloc(&sink, 8));
  cudaEvent_t e0, e1;
  CLA_CUDA(cudaEventCreate(&e0));
  CLA_CUDA(cudaEventCreate(&e1));
  const int blocks = prop.multiProcessorCount * 4, threads = 256, iters = 20000;
  float ms = 0;
  for (int pass = 0; pass < 2; pass++) {  // first pass warms up
    CLA_CUDA(cudaEventRecord(e0));
    k_peak_dmma<<<blocks, threads>>>(iters, sink);
    CLA_CUDA(cudaEventRecord(e1));
    CLA_CUDA(cudaEventSynchronize(e1));
    CLA_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  }
  *dmmaTflops = (double)blocks * (threads / 32) * iters * 8.0 * 512.0 / (ms * 1e-3) / 1e12;
  for (int pass = 0; pass < 2; pass++) {
    CLA_CUDA(cudaEventRecord(e0));
    k_peak_dfma<<<blocks, threads>>>(iters, sink);
    CLA_CUDA(cudaEventRecord(e1));
    CLA_CUDA(cudaEventSynchronize(e1));
    CLA_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  }
  *dfmaTflops = (double)blocks * threads * iters * 16.0 * 2.0 / (ms * 1e-3) / 1e12;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(sink);
  return CLA_OK;
}

// The 16-warp kernel is instantiated for the map widths the decode specialises on and, by tile slots per warp, for
// 3, 6 and 9 slots of 8 x 8 tiles (up to 48, 104 and 128 columns; rows read from a decompressed chunk) and for 2 and 5
// slots of 16 x 8 tiles (up to 64 and 128 columns; decoded on the fly).
template <int TPW>
static void tri16_go(bool fused, int mt, int simple, int grid, size_t smem, cudaStream_t s, const DevGroup* groups,
                     const int32_t* colSrc, const double* constV, const double* X, int rows, int n, double* dOut, int32_t* err) {
#define TRI16(F, M, S) k_tsmm_tri16<F, M, TPW, S><<<grid, T16_THREADS, smem, s>>>(groups, colSrc, constV, X, 0, rows, n, dOut, err)
  if (!fused) TRI16(false, -2, 0);
  else if (mt == CLA_MAP_BYTE && simple == 1) TRI16(true, CLA_MAP_BYTE, 1);
  else if (mt == CLA_MAP_BYTE && simple == 2) TRI16(true, CLA_MAP_BYTE, 2);
  else if (mt == CLA_MAP_CHAR && simple == 1) TRI16(true, CLA_MAP_CHAR, 1);
  else if (mt == CLA_MAP_CHAR && simple == 2) TRI16(true, CLA_MAP_CHAR, 2);
  else if (mt == CLA_MAP_BYTE) TRI16(true, CLA_MAP_BYTE, 0);
  else if (mt == CLA_MAP_CHAR) TRI16(true, CLA_MAP_CHAR, 0);
  else TRI16(true, -2, 0);
#undef TRI16
}
static void launch_tri16(bool fused, int mt, int simple, int n, int grid, size_t smem, cudaStream_t s, const DevGroup* groups,
                         const int32_t* colSrc, const double* constV, const double* X, int rows, double* dOut, int32_t* err) {
  const int NT = (n + 7) / 8, NI = (n + 15) / 16, perWarp = (NI * NT - NI * (NI - 1) + T16_WARPS - 1) / T16_WARPS;
  if (perWarp <= 2) tri16_go<2>(fused, mt, simple, grid, smem, s, groups, colSrc, constV, X, rows, n, dOut, err);
  else if (perWarp <= 4) tri16_go<4>(fused, mt, simple, grid, smem, s, groups, colSrc, constV, X, rows, n, dOut, err);
  else tri16_go<5>(fused, mt, simple, grid, smem, s, groups, colSrc, constV, X, rows, n, dOut, err);
}
template <int TPW>
static int64_t tri16_set_smem_t(int bytes) {
#define TRI16_ATTR(F, M, S) \
  CLA_CUDA(cudaFuncSetAttribute(k_tsmm_tri16<F, M, TPW, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes))
  TRI16_ATTR(true, -2, 0);
  TRI16_ATTR(true, CLA_MAP_BYTE, 0);
  TRI16_ATTR(true, CLA_MAP_CHAR, 0);
  TRI16_ATTR(true, CLA_MAP_BYTE, 1);
  TRI16_ATTR(true, CLA_MAP_CHAR, 1);
  TRI16_ATTR(true, CLA_MAP_BYTE, 2);
  TRI16_ATTR(true, CLA_MAP_CHAR, 2);
  TRI16_ATTR(false, -2, 0);
#undef TRI16_ATTR
  return CLA_OK;
}
static int64_t tri16_set_smem(int bytes) {
  int64_t rc;
  if ((rc = tri16_set_smem_t<2>(bytes)) < 0) return rc;
  if ((rc = tri16_set_smem_t<4>(bytes)) < 0) return rc;
  return tri16_set_smem_t<5>(bytes);
}

int64_t launch_tsmm(Matrix* m, double* dOut, cudaStream_t s) {
  const int n = m->nCols;
  if (n == 0) return CLA_OK;
  if (m->nRows > 0 && pairs_eligible(m, m, true)) {  // few co-coded groups: on the dictionaries
    const int64_t rc = launch_pairs(m, m, true, dOut, s);
    if (rc < 0) return rc;
    // overlapping groups add to a cell from several pairs, in no fixed order: copy the upper triangle down
    k_mirror<<<std::max(1, std::min(1024, (int)(((int64_t)n * n + 255) / 256))), 256, 0, s>>>(dOut, n);
    m->stats.kernel_launches++;
    CLA_CUDA(cudaGetLastError());
    return CLA_OK;
  }
  CLA_CUDA(cudaMemsetAsync(dOut, 0, sizeof(double) * (size_t)n * n, s));
  if (m->nRows == 0) return CLA_OK;
  int64_t rc;
  const bool tri = n <= 128;
  bool denseOnly = m->colSrcValid;
  for (auto& g : m->groups) denseOnly &= (g.type == GT_DDC || g.type == GT_UNC);
  const size_t tri16Smem = (size_t)((n + 15) / 16 * 16) * (4 * TT_LDB * sizeof(double) + sizeof(TsmmCol) + 28) + 4 * sizeof(uint64_t);
  static bool attrSet[64] = {};  // per device: function attributes belong to the device's context
  bool& attr = attrSet[m->device & 63];
  if (!attr) {
    if ((rc = tri16_set_smem(128 * (4 * TT_LDB * 8 + (int)sizeof(TsmmCol) + 28) + 32)) < 0) return rc;
    attr = true;
  }
  if (tri && denseOnly) {  // one launch over all rows, decoding as it goes
    const int64_t nStages = ((int64_t)m->nRows + TT_KT - 1) / TT_KT;
    // one map width for every column (and every column held by a dense-map group): the specialised decode
    int mt = -1;
    for (auto& g : m->groups) {
      const int w = (g.type != GT_DDC) ? -2
                    : (g.mapType == CLA_MAP_UBYTE || g.mapType == CLA_MAP_BYTE) ? CLA_MAP_BYTE
                    : (g.mapType == CLA_MAP_CHAR ? CLA_MAP_CHAR : -2);
      mt = (mt == -1 || mt == w) ? w : -2;
    }
    // the compact records: every column in exactly one dense-map group of that width (1: single-column groups
    // and no constant part; 2: any group width, constants allowed)
    int simple = 0;
    if (mt == CLA_MAP_BYTE || mt == CLA_MAP_CHAR) {
      int covered = 0;
      bool single = true;
      for (auto& g : m->groups) {
        covered += g.gCols;
        single &= g.gCols == 1;
      }
      if (covered == n) simple = (single && !m->hasConst) ? 1 : 2;  // colSrcValid: no column is counted twice
    }
    prof_begin(m, s);
    launch_tri16(true, mt, simple, n, (int)std::min<int64_t>(m->smCount, nStages), tri16Smem, s, m->dGroups, m->dColSrc,
                 m->hasConst ? m->dConstV : nullptr, nullptr, m->nRows, dOut, m->dErr);
    prof_end(m, s);
    m->stats.kernel_launches++;
  } else {
    // chunk of rows whose dense form stays well inside L2 (48 MB)
    int64_t chunk = (48ll << 20) / ((int64_t)n * 8);
    chunk = std::max<int64_t>(SKIP_ROWS, (chunk / SKIP_ROWS) * SKIP_ROWS);
    chunk = std::min<int64_t>(chunk, ((int64_t)m->nRows + SKIP_ROWS - 1) / SKIP_ROWS * SKIP_ROWS);
    if ((rc = ensure_scratch2(m, (size_t)chunk * n * sizeof(double))) < 0) return rc;
    double* X = (double*)m->scratch2;
    const int nBlk = (n + TS_BLK - 1) / TS_BLK;
    const int nPairs = nBlk * (nBlk + 1) / 2;
    for (int64_t r0 = 0; r0 < m->nRows; r0 += chunk) {
      const int r1 = (int)std::min<int64_t>(m->nRows, r0 + chunk);
      if ((rc = launch_decompress_range(m, (int)r0, r1, X, s)) < 0) return rc;
      const int rows = r1 - (int)r0;
      if (tri) {
        const int64_t nStages = ((int64_t)rows + TT_KT - 1) / TT_KT;
        launch_tri16(false, -2, 0, n, (int)std::min<int64_t>(m->smCount, nStages), tri16Smem, s, nullptr, nullptr, nullptr,
                     X, rows, dOut, m->dErr);
      } else {
        int splits = std::max(1, std::min((rows + TS_KT * 8 - 1) / (TS_KT * 8), (4 * m->smCount + nPairs - 1) / nPairs));
        int rowsPerSplit = ((rows + splits - 1) / splits + GT_KT - 1) / GT_KT * GT_KT;
        splits = (rows + rowsPerSplit - 1) / rowsPerSplit;
        dim3 grid(nPairs, splits);
        k_gemm_tn_dmma<true><<<grid, TS_THREADS, 0, s>>>(X, n, X, n, rows, nBlk, dOut, rowsPerSplit);
      }
      m->stats.kernel_launches++;
    }
  }
  k_mirror<<<std::max(1, std::min(1024, (int)(((int64_t)n * n + 255) / 256))), 256, 0, s>>>(dOut, n);
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

// t(L) %*% R for two compressed matrices over the same rows (CLALibLeftMultBy.leftMultByMatrixTransposed on two
// compressed blocks, lib/CLALibLeftMultBy.java:100-112,170-284). Both sides are decompressed one L2-sized row
// chunk at a time (constants included, so no rank-1 corrections are needed) and the chunks are multiplied on
// the FP64 tensor cores; the dense forms never reach HBM-sized buffers.
int64_t launch_tmm(Matrix* L, Matrix* R, double* dOut, cudaStream_t s) {
  const int a = L->nCols, b = R->nCols;
  if ((int64_t)a * b == 0) return CLA_OK;
  if (L->nRows > 0 && pairs_eligible(L, R, false)) return launch_pairs(L, R, false, dOut, s);  // pair pre-aggregation
  CLA_CUDA(cudaMemsetAsync(dOut, 0, sizeof(double) * (size_t)a * b, s));
  if (L->nRows == 0) return CLA_OK;
  int64_t rc;
  int64_t chunk = (48ll << 20) / ((int64_t)(a + b) * 8);
  chunk = std::max<int64_t>(SKIP_ROWS, (chunk / SKIP_ROWS) * SKIP_ROWS);
  chunk = std::min<int64_t>(chunk, ((int64_t)L->nRows + SKIP_ROWS - 1) / SKIP_ROWS * SKIP_ROWS);
  if ((rc = ensure_scratch2(L, (size_t)chunk * a * sizeof(double))) < 0) return rc;
  if ((rc = ensure_scratch2(R, (size_t)chunk * b * sizeof(double))) < 0) return rc;
  double* XL = (double*)L->scratch2;
  double* XR = (double*)R->scratch2;
  const int nBlkA = (a + TS_BLK - 1) / TS_BLK, nBlkB = (b + TS_BLK - 1) / TS_BLK;
  const int nBlocks = nBlkA * nBlkB;
  for (int64_t r0 = 0; r0 < L->nRows; r0 += chunk) {
    const int r1 = (int)std::min<int64_t>(L->nRows, r0 + chunk);
    if ((rc = launch_decompress_range(L, (int)r0, r1, XL, s)) < 0) return rc;
    if ((rc = launch_decompress_range(R, (int)r0, r1, XR, s)) < 0) return rc;
    const int rows = r1 - (int)r0;
    int splits = std::max(1, std::min((rows + TS_KT * 8 - 1) / (TS_KT * 8), (4 * L->smCount + nBlocks - 1) / nBlocks));
    int rowsPerSplit = ((rows + splits - 1) / splits + GT_KT - 1) / GT_KT * GT_KT;
    splits = (rows + rowsPerSplit - 1) / rowsPerSplit;
    dim3 grid(nBlocks, splits);
    if (r0 == 0) prof_begin(L, s);
    k_gemm_tn_dmma<false><<<grid, TS_THREADS, 0, s>>>(XL, a, XR, b, rows, nBlkB, dOut, rowsPerSplit);
    if (r0 == 0) prof_end(L, s);
    L->stats.kernel_launches++;
  }
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

}  // namespace cla
