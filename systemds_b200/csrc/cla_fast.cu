// Specialised vector products for matrices whose product groups are all dense-map (DDC) groups with
// at most 256 dictionary tuples and one byte per map cell -- the shape of the headline workloads
// (X %*% v, t(y) %*% X and the two passes of t(X) %*% (X %*% v)).
//
// Both kernels are bound by shared-memory lookups (one 8-byte dictionary read per map cell), so the
// layouts are chosen to make those reads bank-conflict free:
//
//  * k_rmm_vec_u8: a thread owns 16 consecutive rows (one 128-bit map load per group) and keeps their
//    16 partial sums in registers; the tables P_g = D_g * v[cols_g] (built per call by k_fast_ptable)
//    sit in shared memory back to back. A table of <= 16 entries spans each 8-byte bank once, so random
//    ids never conflict; larger tables conflict in proportion to their size.
//
//  * k_lmm_vec_u8: a lane owns *columns*, not rows. Tables are interleaved 16 columns wide, one such
//    "unit" after the other (entry k of slot s of a unit at byte k*128 + s*8), so lane s only ever touches
//    bank pair s whatever the ids are: conflict free for any cardinality, without replicating tables. The
//    two half-warps of a warp work on different rows of the same 16 column slots per unit; a CTA holds up
//    to seven units (7 x 32 KB at 256 tuples). The left vector is read with warp-uniform 128-bit loads and
//    kept in registers for all columns of the CTA.
//
// Tables are staged into shared memory with TMA bulk copies (cp.async.bulk + mbarrier, no multicast).
#include "cla_common.cuh"
#include <algorithm>
#include <cstdlib>
#include <numeric>

namespace cla {

int64_t launch_lmm_const(Matrix* m, const double* dYt, int q, double* dOut, cudaStream_t s);  // cla_generic.cu
int64_t launch_lmm_const_with(Matrix* m, const double* dYt, int q, double* dOut, double* sums, cudaStream_t s);

constexpr int FAST_MIN_ROWS = 4096;
constexpr int SMEM_MAX = 227 * 1024;

// ---- RMM plan ----
constexpr int RMM_T = 128;            // threads (128 / 256 / 512 measured on 10M x 100, 16 values: 0.313 / 0.320 / 0.496 ms)
constexpr int RMM_ROWS_PT = 16;       // rows per thread
constexpr int RMM_TILE = RMM_T * RMM_ROWS_PT;

// ---- LMM plan ----
// Warps per CTA (one CTA per SM). Measured on the benchmark workloads for 10 / 12 / 14 / 16 warps: t(y) X 10M x 200
// 0.718 / 0.675 / 0.682 / 0.654 ms (sixteen warps fit 128 registers with 20 bytes of spills), the fused X v 1M x 100
// 0.0699 / 0.0686 / 0.0688 / 0.0665 ms per step; k_rmm_vec_b is the exception (lmCG step 9.32 / 8.52 / 8.51 / 8.56 ms).
constexpr int LMM_W = 16;
constexpr int LMM_T = LMM_W * 32;
constexpr int RB_W = 12;              // k_rmm_vec_b
constexpr int LMM_MAX_UNITS = 7;      // 16-column table units per CTA (7 x 32 KB at 256 tuples)
constexpr int LMM_PART = LMM_MAX_UNITS * 16;  // partial sums a CTA writes
constexpr int LMM_STEP = 64;          // rows per warp step (32 per half-warp)

struct RmmChunk {
  int g0, g1;          // range in plan order
  int tblDoubles;      // table doubles of the chunk (even)
  int64_t tblOff;      // offset of the chunk's tables in the P image (doubles, even)
};
struct LmmChunk {
  int unit0, nUnits;     // units of 16 column slots
  int nk[LMM_MAX_UNITS]; // table depth (max tuples) of each unit
  int64_t tblOff;        // offset in the table image (doubles)
  int tblDoubles;
  int cta0, nCta;        // CTA range of the launch that works on this chunk
};

struct FastPlan {
  bool ok = false;
  bool partial = false;  // only some groups are covered; the general kernels add the rest
  int nG = 0;
  // RMM
  std::vector<RmmChunk> rchunks;
  const uint8_t** dMaps = nullptr;  // [nG] plan order
  int* dTblOff = nullptr;           // [nG] offset of each group's table inside its chunk (doubles)
  int* dGroupOf = nullptr;          // [nG] plan order -> device group index
  int64_t* dImgOff = nullptr;       // [nG] offset of each group's table in the P image (doubles)
  int64_t pImgDoubles = 0;
  // LMM
  int nUnits = 0, nSlots = 0;
  std::vector<LmmChunk> lchunks;
  LmmChunk* dLChunks = nullptr;
  const uint8_t** dSlotMap = nullptr;  // [nSlots] column-major byte maps (plan order)
  uint8_t* dLmmMaps = nullptr;         // the same maps interleaved for the column-per-lane kernel (see k_lmm_interleave)
  int64_t nRB = 0;                     // 16-row blocks per column in that layout (padded to whole 64-row steps)
  int* dSlotCol = nullptr;             // [nSlots] output column or -1
  double* dLmmTables = nullptr;        // image of all chunk tables
  int lmmGrid = 0;
  int maxNVals = 0;                    // deepest table: <= 16 keeps the row-per-thread kernel conflict free
  size_t imageDoubles = 0;
  // RMM with two groups per lookup (small dictionaries): see k_rmm_vec_f
  bool fusedOk = false;
  int nFused = 0;
  std::vector<LmmChunk> fchunks;
  LmmChunk* dFChunks = nullptr;
  struct FusedUnit* dFUnits = nullptr;  // [slots]
  uint8_t* dFMaps = nullptr;            // [slab16][16-row block][a | b][slot][16 ids]
  size_t fImageDoubles = 0;
  std::vector<void*> allocs;
};

// One column slot of the fused RMM: ids a (group ga) and b (group gb, or none) of a row address entry (a << sh) | b.
struct FusedUnit {
  int32_t ga, gb;   // device group indices, gb = -1: no second group
  int32_t sh;       // bits reserved for b
  int32_t nva, nvb;
};

// --------------------------------------------------------------------------------------------------
// TMA bulk copy global -> shared, completion on an mbarrier; bounded wait.
// --------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Copies `bytes` (multiple of 16, both addresses 16-byte aligned) and waits. Returns false on timeout.
__device__ __forceinline__ bool tma_load_to_smem(void* dst, const void* src, uint32_t bytes, uint64_t* mbar) {
  const uint32_t bar = smem_u32(mbar);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    const uint32_t CH = 32768;
    for (uint32_t off = 0; off < bytes; off += CH) {
      const uint32_t sz = min(CH, bytes - off);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       smem_u32((char*)dst + off)),
                   "l"((const char*)src + off), "r"(sz), "r"(bar)
                   : "memory");
    }
  }
  uint32_t done = 0;
  for (int it = 0; it < (1 << 22) && !done; it++) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(0u)
        : "memory");
  }
  // one verdict for the whole CTA (also the barrier that publishes the data to every thread)
  return __syncthreads_and(done != 0) != 0;
}

// The same copy for kernels that reload the buffer several times: the barrier is initialised once and each use
// waits on the next phase parity. The caller must have synchronised the CTA (all reads of the old contents done)
// before calling; the issuing thread then orders those generic-proxy reads before the async-proxy writes.
__device__ __forceinline__ void tma_barrier_init(uint64_t* mbar) {
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(mbar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
}
__device__ __forceinline__ bool tma_reload(void* dst, const void* src, uint32_t bytes, uint64_t* mbar, uint32_t parity) {
  const uint32_t bar = smem_u32(mbar);
  if (threadIdx.x == 0) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    const uint32_t CH = 32768;
    for (uint32_t off = 0; off < bytes; off += CH) {
      const uint32_t sz = min(CH, bytes - off);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       smem_u32((char*)dst + off)),
                   "l"((const char*)src + off), "r"(sz), "r"(bar)
                   : "memory");
    }
  }
  uint32_t done = 0;
  for (int it = 0; it < (1 << 22) && !done; it++) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
  }
  return __syncthreads_and(done != 0) != 0;
}

// --------------------------------------------------------------------------------------------------
// RMM: P image (padded per-group tables), then the row kernel
// --------------------------------------------------------------------------------------------------
__global__ void k_fast_ptable(const DevGroup* __restrict__ groups, const int* __restrict__ groupOf,
                              const int64_t* __restrict__ imgOff, int nG, const double* __restrict__ v,
                              double* __restrict__ P) {
  const int gi = blockIdx.x;
  if (gi >= nG) return;
  const DevGroup& g = groups[groupOf[gi]];
  for (int k = threadIdx.x; k < g.nVals; k += blockDim.x) {
    double s = 0;
    for (int h = 0; h < g.gCols; h++) s += g.dict[(size_t)k * g.gCols + h] * v[g.cols[h]];
    P[imgOff[gi] + k] = s;
  }
}

__device__ __forceinline__ uint32_t byte_x8(uint32_t w, int i) {  // (byte i of w) * 8
  return i == 0 ? (w << 3) & 0x7F8u : (w >> (8 * i - 3)) & 0x7F8u;
}

template <int R>
struct MapWord;
template <> struct MapWord<16> { typedef uint4 T; };
template <> struct MapWord<8> { typedef uint2 T; };
template <> struct MapWord<4> { typedef uint32_t T; };

// R = rows per thread (16, 8 or 4): fewer rows per thread means more threads for short matrices.
template <int R>
__global__ void __launch_bounds__(RMM_T)
k_rmm_vec_u8(const uint8_t* const* __restrict__ maps, const int* __restrict__ tblOff, int g0, int g1,
             const double* __restrict__ Pchunk, int tblDoubles, int nRows, const double* __restrict__ constRow,
             double* __restrict__ out, int accumulate, int32_t* err) {
  extern __shared__ __align__(128) unsigned char smraw[];
  double* tables = (double*)smraw;
  const int nG = g1 - g0;
  const uint8_t** sMaps = (const uint8_t**)(smraw + (size_t)tblDoubles * 8);
  int* sOff = (int*)(sMaps + nG);
  __shared__ __align__(8) uint64_t mbar;
  const int tid = threadIdx.x;
  for (int i = tid; i < nG; i += RMM_T) {
    sMaps[i] = maps[g0 + i];
    sOff[i] = tblOff[g0 + i] * 8;  // byte offset
  }
  if (!tma_load_to_smem(tables, Pchunk, (uint32_t)tblDoubles * 8u, &mbar)) {
    if (tid == 0) atomicExch(err, 100);
    return;
  }
  const double c0 = (constRow != nullptr && !accumulate) ? constRow[0] : 0.0;
  constexpr int TILE = RMM_T * R;
  const int nTiles = (nRows + TILE - 1) / TILE;
  const unsigned char* tb = (const unsigned char*)tables;
  typedef typename MapWord<R>::T W;
  for (int tile = blockIdx.x; tile < nTiles; tile += gridDim.x) {
    const int row = tile * TILE + tid * R;
    if (row >= nRows) continue;
    if (row + R <= nRows) {
      double acc[R];
#pragma unroll
      for (int i = 0; i < R; i++) acc[i] = c0;
#pragma unroll(R == 16 ? 8 : 16)
      for (int g = 0; g < nG; g++) {
        const W w = __ldg((const W*)(sMaps[g] + row));
        const unsigned char* T = tb + sOff[g];
        uint32_t ww[4];
        if constexpr (R == 16) { ww[0] = w.x; ww[1] = w.y; ww[2] = w.z; ww[3] = w.w; }
        else if constexpr (R == 8) { ww[0] = w.x; ww[1] = w.y; }
        else { ww[0] = w; }
#pragma unroll
        for (int i = 0; i < R; i++) acc[i] += *(const double*)(T + byte_x8(ww[i >> 2], i & 3));
      }
      if (accumulate) {
#pragma unroll
        for (int i = 0; i < R; i++) atomicAdd(out + row + i, acc[i]);
      } else {
        double2* o = (double2*)(out + row);
#pragma unroll
        for (int i = 0; i < R / 2; i++) o[i] = make_double2(acc[2 * i], acc[2 * i + 1]);
      }
    } else {  // ragged last rows
      for (int r = row; r < nRows; r++) {
        double a = c0;
        for (int g = 0; g < nG; g++) a += *(const double*)(tb + sOff[g] + 8 * (int)sMaps[g][r]);
        if (accumulate) atomicAdd(out + r, a);
        else out[r] = a;
      }
    }
  }
}

// --------------------------------------------------------------------------------------------------
// LMM: column-per-lane kernel
// --------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t byte_x128(uint32_t w, int i) {  // (byte i of w) << 7
  return i == 0 ? (w << 7) & 0x7F80u : (i == 3 ? (w >> 17) & 0x7F80u : (w >> (8 * i - 7)) & 0x7F80u);
}

template <int NU>
__device__ __forceinline__ void lmm_cells(const uint4 (&m)[NU][2], int sub, const double (&yv)[16],
                                          const unsigned char* const (&tbase)[NU], double (&acc)[NU]) {
#pragma unroll
  for (int u = 0; u < NU; u++) {
    const uint4 w = m[u][sub];
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    const unsigned char* T = tbase[u];
#pragma unroll
    for (int i = 0; i < 16; i++) {
      const double t = *(const double*)(T + byte_x128(ww[i >> 2], i & 3));
      acc[u] = fma(yv[i], t, acc[u]);
    }
  }
}

// partial: [gridDim.x][LMM_PART]
template <int NU>
__device__ __forceinline__ void lmm_vec_body(const LmmChunk& ch, const uint8_t* __restrict__ imaps, int64_t nRB,
                                             const double* __restrict__ tablesImg, const double* __restrict__ y,
                                             int nRows, int64_t stepBegin, int64_t stepEnd,
                                             double* __restrict__ partial, unsigned char* smraw, uint64_t* mbar,
                                             int32_t* err) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = lane & 15, half = lane >> 4;
  if (!tma_load_to_smem(smraw, tablesImg + ch.tblOff, (uint32_t)ch.tblDoubles * 8u, mbar)) {
    // the tables never arrived: flag it, and make the failure visible in the result as well (the final kernel sums
    // this row whatever happens, and a device-buffer caller only sees the error word at its next cla_stats_get)
    if (tid == 0) atomicExch(err, 101);
    for (int u = tid; u < NU * 16; u += LMM_T) partial[(size_t)blockIdx.x * LMM_PART + u] = __longlong_as_double(0x7ff8000000000000ll);
    return;
  }
  // table base of each unit for this lane (slot offset folded in), and this lane's map pointers
  const unsigned char* tbase[NU];
  const uint8_t* mp[NU];
  {
    size_t off = 0;
#pragma unroll
    for (int u = 0; u < NU; u++) {
      tbase[u] = smraw + off + slot * 8;
      off += (size_t)ch.nk[u] * 128;
      mp[u] = imaps + (size_t)(ch.unit0 + u) * nRB * 256 + slot * 16;
    }
  }
  double acc[NU];
#pragma unroll
  for (int u = 0; u < NU; u++) acc[u] = 0.0;

  // rows of this CTA: contiguous range of 64-row steps
  const int ctaInChunk = blockIdx.x - ch.cta0;
  const int64_t nSteps = stepEnd - stepBegin;  // this launch covers the 64-row steps [stepBegin, stepEnd)
  const int64_t s0 = stepBegin + nSteps * ctaInChunk / ch.nCta, s1 = stepBegin + nSteps * (ctaInChunk + 1) / ch.nCta;
  for (int64_t st = s0 + warp; st < s1; st += LMM_W) {
    const int64_t r0 = st * LMM_STEP + half * 32;
    if (st * LMM_STEP + LMM_STEP <= nRows) {
      uint4 m[NU][2];
#pragma unroll
      for (int u = 0; u < NU; u++) {
        const uint8_t* src = mp[u] + (r0 >> 4) * 256;
        m[u][0] = __ldg((const uint4*)src);
        m[u][1] = __ldg((const uint4*)(src + 256));
      }
#pragma unroll
      for (int sub = 0; sub < 2; sub++) {
        double yv[16];
        const double2* ys = (const double2*)(y + r0 + sub * 16);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const double2 t = __ldg(ys + i);
          yv[2 * i] = t.x;
          yv[2 * i + 1] = t.y;
        }
        lmm_cells<NU>(m, sub, yv, tbase, acc);
      }
    } else {  // ragged last step
      for (int64_t r = r0; r < min((int64_t)nRows, r0 + 32); r++) {
        const double yy = y[r];
#pragma unroll
        for (int u = 0; u < NU; u++)
          acc[u] = fma(yy, *(const double*)(tbase[u] + 128 * (int)mp[u][(r >> 4) * 256 + (r & 15)]), acc[u]);
      }
    }
  }
  // combine the two half-warps (same column slots, different rows), then the warps through shared memory
  __syncthreads();  // tables no longer needed
  double* red = (double*)smraw;  // [LMM_W][NU*16]
#pragma unroll
  for (int u = 0; u < NU; u++) {
    double a = acc[u];
    a += __shfl_xor_sync(0xffffffffu, a, 16);
    if (half == 0) red[warp * (NU * 16) + u * 16 + slot] = a;
  }
  __syncthreads();
  for (int u = tid; u < NU * 16; u += LMM_T) {
    double s = 0;
    for (int w = 0; w < LMM_W; w++) s += red[w * (NU * 16) + u];
    partial[(size_t)blockIdx.x * LMM_PART + u] = s;
  }
}

__global__ void __launch_bounds__(LMM_T, 1)
k_lmm_vec_u8(const LmmChunk* __restrict__ chunks, int nChunks, const uint8_t* __restrict__ imaps, int64_t nRB,
             const double* __restrict__ tablesImg, const double* __restrict__ y, int nRows, int64_t stepBegin,
             int64_t stepEnd, double* __restrict__ partial, int32_t* err) {
  extern __shared__ __align__(128) unsigned char smraw[];
  __shared__ __align__(8) uint64_t mbar;
  __shared__ LmmChunk ch;
  if (threadIdx.x == 0) {
    int c = 0;
    while (c + 1 < nChunks && (int)blockIdx.x >= chunks[c].cta0 + chunks[c].nCta) c++;
    ch = chunks[c];
  }
  __syncthreads();
#define LMM_CASE(N) case N: lmm_vec_body<N>(ch, imaps, nRB, tablesImg, y, nRows, stepBegin, stepEnd, partial, smraw, &mbar, err); break;
  switch (ch.nUnits) {
    LMM_CASE(1) LMM_CASE(2) LMM_CASE(3) LMM_CASE(4) LMM_CASE(5) LMM_CASE(6)
    default: lmm_vec_body<7>(ch, imaps, nRB, tablesImg, y, nRows, stepBegin, stepEnd, partial, smraw, &mbar, err); break;
  }
#undef LMM_CASE
}

// out[col] += sum over the chunk's CTAs of partial[cta][slot]. A warp per column slot: lane l adds the partial sums of
// CTAs l, l + 32, ... (row ranges that were launched separately one after the other), then a shuffle tree adds the
// 32 lanes -- a fixed order for a given launch geometry, so the result is reproducible, and the 80 or so partial
// sums of a column are no longer one chain of dependent loads.
__global__ void k_lmm_vec_final(const LmmChunk* __restrict__ chunks, int nChunks, const int* __restrict__ slotCol,
                                const double* __restrict__ partial, double* __restrict__ out, int nParts, int gridPerPart) {
  const int c = blockIdx.x;
  if (c >= nChunks) return;
  const LmmChunk ch = chunks[c];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nWarps = (blockDim.x >> 5) * gridDim.y;
  const int n = nParts * ch.nCta;
  for (int u = blockIdx.y * (blockDim.x >> 5) + warp; u < ch.nUnits * 16; u += nWarps) {  // gridDim.y CTAs per chunk
    const int col = slotCol[ch.unit0 * 16 + u];
    if (col < 0) continue;
    double s = 0;
    for (int i = lane; i < n; i += 32) {
      const int part = i / ch.nCta, b = i - part * ch.nCta;
      s += partial[((size_t)part * gridPerPart + ch.cta0 + b) * LMM_PART + u];
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    if (lane == 0) atomicAdd(&out[col], s);
  }
}

// --------------------------------------------------------------------------------------------------
// LMM with Q left rows at once (Q = 2 or 4; the reference's left-multiply blocks four rows too,
// lib/CLALibLeftMultBy.java:731-819). Same layout and lookups as k_lmm_vec_u8, but a dictionary value fetched for a
// cell multiplies the cell's Q left values: one pass over the maps and one lookup per cell serve Q rows, where Q
// passes of the one-row kernel would fetch each value Q times. partial: [gridDim.x][Q][LMM_PART].
// --------------------------------------------------------------------------------------------------
constexpr int LQ_W = 12;              // warps per CTA (Q x NU accumulators per lane: up to 170 registers)
constexpr int LQ_T = LQ_W * 32;

template <int NU, int Q>
__device__ __forceinline__ void lmmq_body(const LmmChunk& ch, const uint8_t* __restrict__ imaps, int64_t nRB,
                                          const double* __restrict__ tablesImg, const double* __restrict__ y, size_t pitch,
                                          int nRows, double* __restrict__ partial, unsigned char* smraw, uint64_t* mbar,
                                          int32_t* err) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = lane & 15, half = lane >> 4;
  if (!tma_load_to_smem(smraw, tablesImg + ch.tblOff, (uint32_t)ch.tblDoubles * 8u, mbar)) {
    if (tid == 0) atomicExch(err, 105);
    for (int u = tid; u < Q * LMM_PART; u += LQ_T) partial[(size_t)blockIdx.x * Q * LMM_PART + u] = __longlong_as_double(0x7ff8000000000000ll);
    return;
  }
  const unsigned char* tbase[NU];
  const uint8_t* mp[NU];
  {
    size_t off = 0;
#pragma unroll
    for (int u = 0; u < NU; u++) {
      tbase[u] = smraw + off + slot * 8;
      off += (size_t)ch.nk[u] * 128;
      mp[u] = imaps + (size_t)(ch.unit0 + u) * nRB * 256 + slot * 16;
    }
  }
  double acc[NU][Q];
#pragma unroll
  for (int u = 0; u < NU; u++)
#pragma unroll
    for (int q = 0; q < Q; q++) acc[u][q] = 0.0;
  const int ctaInChunk = blockIdx.x - ch.cta0;
  const int64_t nSteps = ((int64_t)nRows + LMM_STEP - 1) / LMM_STEP;
  const int64_t s0 = nSteps * ctaInChunk / ch.nCta, s1 = nSteps * (ctaInChunk + 1) / ch.nCta;
  for (int64_t st = s0 + warp; st < s1; st += LQ_W) {
    const int64_t r0 = st * LMM_STEP + half * 32;
    if (st * LMM_STEP + LMM_STEP <= nRows) {
#pragma unroll 1
      for (int sub = 0; sub < 2; sub++) {
        uint4 m[NU];
#pragma unroll
        for (int u = 0; u < NU; u++) m[u] = __ldg((const uint4*)(mp[u] + ((r0 >> 4) + sub) * 256));
        const double* yr = y + r0 + sub * 16;
#pragma unroll
        for (int i = 0; i < 16; i += 2) {  // two rows per 128-bit load of every left row
          double2 yq[Q];
#pragma unroll
          for (int q = 0; q < Q; q++) yq[q] = __ldg((const double2*)(yr + q * pitch + i));
#pragma unroll
          for (int u = 0; u < NU; u++) {
            const uint32_t w = (i >> 2) == 0 ? m[u].x : ((i >> 2) == 1 ? m[u].y : ((i >> 2) == 2 ? m[u].z : m[u].w));
            const double t0 = *(const double*)(tbase[u] + byte_x128(w, i & 3));
            const double t1 = *(const double*)(tbase[u] + byte_x128(w, (i & 3) + 1));
#pragma unroll
            for (int q = 0; q < Q; q++) acc[u][q] = fma(yq[q].y, t1, fma(yq[q].x, t0, acc[u][q]));
          }
        }
      }
    } else {  // ragged last step
      for (int64_t r = r0; r < min((int64_t)nRows, r0 + 32); r++) {
#pragma unroll
        for (int u = 0; u < NU; u++) {
          const double t = *(const double*)(tbase[u] + 128 * (int)mp[u][(r >> 4) * 256 + (r & 15)]);
#pragma unroll
          for (int q = 0; q < Q; q++) acc[u][q] = fma(y[q * pitch + r], t, acc[u][q]);
        }
      }
    }
  }
  __syncthreads();  // tables no longer needed
  double* red = (double*)smraw;  // [LQ_W][Q][NU*16]
#pragma unroll
  for (int u = 0; u < NU; u++)
#pragma unroll
    for (int q = 0; q < Q; q++) {
      double a = acc[u][q];
      a += __shfl_xor_sync(0xffffffffu, a, 16);
      if (half == 0) red[(warp * Q + q) * (NU * 16) + u * 16 + slot] = a;
    }
  __syncthreads();
  for (int e = tid; e < Q * NU * 16; e += LQ_T) {
    const int q = e / (NU * 16), u = e - q * (NU * 16);
    double s = 0;
    for (int w = 0; w < LQ_W; w++) s += red[(w * Q + q) * (NU * 16) + u];
    partial[((size_t)blockIdx.x * Q + q) * LMM_PART + u] = s;
  }
}

template <int Q>
__global__ void __launch_bounds__(LQ_T, 1)
k_lmm_vecq_u8(const LmmChunk* __restrict__ chunks, int nChunks, const uint8_t* __restrict__ imaps, int64_t nRB,
              const double* __restrict__ tablesImg, const double* __restrict__ y, size_t pitch, int nRows,
              double* __restrict__ partial, int32_t* err) {
  extern __shared__ __align__(128) unsigned char smraw[];
  __shared__ __align__(8) uint64_t mbar;
  __shared__ LmmChunk ch;
  if (threadIdx.x == 0) {
    int c = 0;
    while (c + 1 < nChunks && (int)blockIdx.x >= chunks[c].cta0 + chunks[c].nCta) c++;
    ch = chunks[c];
  }
  __syncthreads();
#define LQ_CASE(N) case N: lmmq_body<N, Q>(ch, imaps, nRB, tablesImg, y, pitch, nRows, partial, smraw, &mbar, err); break;
  switch (ch.nUnits) {
    LQ_CASE(1) LQ_CASE(2) LQ_CASE(3) LQ_CASE(4) LQ_CASE(5) LQ_CASE(6)
    default: lmmq_body<7, Q>(ch, imaps, nRB, tablesImg, y, pitch, nRows, partial, smraw, &mbar, err); break;
  }
#undef LQ_CASE
}

// out[q][col] += sum over the chunk's CTAs of partial[cta][q][slot]; blockIdx.z = q
__global__ void k_lmm_vecq_final(const LmmChunk* __restrict__ chunks, int nChunks, const int* __restrict__ slotCol,
                                 const double* __restrict__ partial, double* __restrict__ out, int Q, int nCols) {
  const int c = blockIdx.x, q = blockIdx.z;
  if (c >= nChunks) return;
  const LmmChunk ch = chunks[c];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nWarps = (blockDim.x >> 5) * gridDim.y;
  for (int u = blockIdx.y * (blockDim.x >> 5) + warp; u < ch.nUnits * 16; u += nWarps) {
    const int col = slotCol[ch.unit0 * 16 + u];
    if (col < 0) continue;
    double s = 0;
    for (int i = lane; i < ch.nCta; i += 32) s += partial[((size_t)(ch.cta0 + i) * Q + q) * LMM_PART + u];
#pragma unroll
    for (int d = 16; d; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    if (lane == 0) atomicAdd(&out[(size_t)q * nCols + col], s);
  }
}

// --------------------------------------------------------------------------------------------------
// Decompress from the column-per-lane layout.
//
// Same chunks, interleaved maps and table images as k_lmm_vec_u8: lane s of a half-warp owns column slot s of a
// unit, loads 16 rows of its ids with one 128-bit load, reads each value from its own bank pair of the unit's
// table and stores it. The 16 slots of a unit are 16 neighbouring output columns (the plan orders the slots by
// column), so a warp store writes two full 128-byte pieces of two rows: no transposition through shared memory,
// no bank conflicts, no gathers from global memory. Per 32 cells the L1 data pipe sees 2 wavefronts of lookups,
// 2 of stores and 1/4 of map loads (the tile kernel in cla_generic.cu needs about 20, most of them for the gather
// of dictionary values through L1), which puts the bound on the output stream. Every cell is written exactly once
// with the same operation as the tile kernel (column constant + dictionary value).
// --------------------------------------------------------------------------------------------------
constexpr int DEC_W = 12;  // warps per CTA (measured 8 / 10 / 12 / 14 / 16 / 20 / 24: 12 writes the most, 4.2-4.5 TB/s)
constexpr int DEC_T = DEC_W * 32;
constexpr int DEC_NP = (LMM_MAX_UNITS + 1) / 2;  // unit pairs of a chunk: a warp store covers 32 neighbouring columns

__global__ void __launch_bounds__(DEC_T, 1)
k_decomp_fast(const LmmChunk* __restrict__ chunks, int nChunks, const uint8_t* __restrict__ imaps, int64_t nRB,
              const double* __restrict__ tablesImg, const int* __restrict__ slotCol, const double* __restrict__ constV,
              double* __restrict__ out, int nCols, int r0, int r1, int32_t* err) {
  extern __shared__ __align__(128) unsigned char smraw[];
  __shared__ __align__(8) uint64_t mbar;
  __shared__ LmmChunk ch;
  __shared__ int unitOff[LMM_MAX_UNITS];
  __shared__ int sCol[LMM_MAX_UNITS * 16];
  __shared__ double sCst[LMM_MAX_UNITS * 16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = lane & 15, half = lane >> 4;
  if (tid == 0) {
    int c = 0;
    while (c + 1 < nChunks && (int)blockIdx.x >= chunks[c].cta0 + chunks[c].nCta) c++;
    ch = chunks[c];
    int off = 0;
    for (int u = 0; u < ch.nUnits; u++) {
      unitOff[u] = off;
      off += ch.nk[u] * 128;
    }
  }
  __syncthreads();
  if (tid < ch.nUnits * 16) {
    const int col = slotCol[ch.unit0 * 16 + tid];
    sCol[tid] = col;
    sCst[tid] = (constV && col >= 0) ? constV[col] : 0.0;
  }
  const int NU = ch.nUnits;
  const int ctaInChunk = blockIdx.x - ch.cta0;
  const int64_t stepBegin = r0 / LMM_STEP, stepEnd = ((int64_t)r1 + LMM_STEP - 1) / LMM_STEP;  // r0 is a multiple of LMM_STEP
  const int64_t nSteps = stepEnd - stepBegin;
  const int64_t s0 = stepBegin + nSteps * ctaInChunk / ch.nCta, s1 = stepBegin + nSteps * (ctaInChunk + 1) / ch.nCta;
  const size_t ld = (size_t)nCols;
  if (!tma_load_to_smem(smraw, tablesImg + ch.tblOff, (uint32_t)ch.tblDoubles * 8u, &mbar)) {
    // the tables never arrived: flag it, and make the failure visible in this CTA's cells as well (a device-buffer
    // caller only sees the error word at its next cla_stats_get)
    if (tid == 0) atomicExch(err, 102);
    const int64_t rb = s0 * LMM_STEP, re = min((int64_t)r1, s1 * LMM_STEP);
    const int w = NU * 16;
    for (int64_t i = tid; i < (re - rb) * w; i += DEC_T) {
      const int col = sCol[(int)(i % w)];
      if (col >= 0) out[(size_t)(rb + i / w - r0) * ld + col] = __longlong_as_double(0x7ff8000000000000ll);
    }
    return;
  }
  // This lane's column of every unit pair: unit 2p + half, slot lane & 15
  int toff[DEC_NP];   // byte offset of the lane's table column in shared memory
  double cst[DEC_NP];
  int colOf[DEC_NP];
#pragma unroll
  for (int p = 0; p < DEC_NP; p++) {
    const int u = 2 * p + half;
    const bool ok = u < NU;
    colOf[p] = ok ? sCol[u * 16 + slot] : -1;
    cst[p] = ok ? sCst[u * 16 + slot] : 0.0;
    toff[p] = (ok ? unitOff[u] : 0) + slot * 8;
  }
  // ids of this lane's column of pair p, 16-row block b: units lie nRB * 256 bytes apart, a missing last unit reads unit 0's
  const uint8_t* mbase = imaps + (size_t)ch.unit0 * nRB * 256 + slot * 16;
  const size_t pairStride = (size_t)2 * nRB * 256, halfOff = (size_t)half * nRB * 256;
  auto ids_at = [&](int p, int64_t b) {
    const size_t uo = (2 * p + half < NU) ? p * pairStride + halfOff : 0;
    return __ldg((const uint4*)(mbase + uo + b * 256));
  };
  // A warp owns 16-row blocks; it writes them a row at a time, 256 contiguous bytes per store and the chunk's columns
  // of a row one after the other: runs of consecutive addresses are what the memory system turns into full-rate
  // writes (the same cells written as 128-byte pieces of many rows reach about 0.9 of this order's rate). The ids of
  // the next block are loaded before the current one is looked up.
  const int64_t b0 = s0 * (LMM_STEP / 16), b1 = s1 * (LMM_STEP / 16);
  uint4 w[DEC_NP], nw[DEC_NP];
  int64_t blk = b0 + warp;
  if (blk < b1) {
#pragma unroll
    for (int p = 0; p < DEC_NP; p++) w[p] = ids_at(p, blk);
  }
  for (; blk < b1; blk += DEC_W) {
    if (blk + DEC_W < b1) {
#pragma unroll
      for (int p = 0; p < DEC_NP; p++) nw[p] = ids_at(p, blk + DEC_W);
    }
    const int64_t row0 = blk * 16;
    double* o = out + (size_t)(row0 - r0) * ld;
    const bool whole = row0 + 16 <= r1;
#pragma unroll 1
    for (int j = 0; j < 4; j++) {  // four rows per round (one id word per unit pair): 4 x DEC_NP lookups in flight
      uint32_t word[DEC_NP];
#pragma unroll
      for (int p = 0; p < DEC_NP; p++) word[p] = j == 0 ? w[p].x : (j == 1 ? w[p].y : (j == 2 ? w[p].z : w[p].w));
      double* orow = o + (size_t)(4 * j) * ld;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        if (whole || row0 + 4 * j + i < r1) {
#pragma unroll
          for (int p = 0; p < DEC_NP; p++)
            if (colOf[p] >= 0) orow[colOf[p]] = cst[p] + *(const double*)(smraw + toff[p] + byte_x128(word[p], i));
        }
        orow += ld;
      }
    }
#pragma unroll
    for (int p = 0; p < DEC_NP; p++) w[p] = nw[p];
  }
}

// --------------------------------------------------------------------------------------------------
// RMM, column-per-lane variant (tables of any depth up to 256 without bank conflicts).
// Same slabs, interleaved maps and table layout as k_lmm_vec_u8; the table of slot s holds
// D[:, j] * v[col] (k_rmm_b_tables), so summing a row's lookups over all slots gives the row of X v.
// A CTA owns a contiguous range of rows and walks the column chunks one after the other, reloading the tables;
// the first chunk stores its partial sums, later chunks add to them (the CTA owns the rows: no atomics, and the
// summation order is fixed). Within a chunk each lane accumulates 16 rows x its column slots, then a
// reduce-scatter over the 16 lanes of the half-warp (15 shuffles) leaves lane s with the sum of row s.
// --------------------------------------------------------------------------------------------------
__global__ void k_rmm_b_tables(const LmmChunk* __restrict__ chunks, const int* __restrict__ slotCol,
                               const double* __restrict__ T, const double* __restrict__ v, double* __restrict__ P) {
  const LmmChunk ch = chunks[blockIdx.x];
  int base = 0;
  for (int u = 0; u < ch.nUnits; u++) {
    const int n = ch.nk[u] * 16;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < n; e += gridDim.y * blockDim.x) {  // gridDim.y CTAs per chunk
      const int col = slotCol[(ch.unit0 + u) * 16 + (e & 15)];
      P[ch.tblOff + base + e] = col >= 0 ? T[ch.tblOff + base + e] * v[col] : 0.0;
    }
    base += n;
  }
}

template <int NU>
__device__ __forceinline__ void rmm_b_chunk(const LmmChunk& ch, const uint8_t* __restrict__ imaps, int64_t nRB,
                                            int64_t s0, int64_t s1, int nRows, double init, bool first,
                                            double* __restrict__ out, const unsigned char* smraw) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slot = lane & 15, half = lane >> 4;
  const unsigned char* tbase[NU];
  const uint8_t* mp[NU];
  {
    size_t off = 0;
#pragma unroll
    for (int u = 0; u < NU; u++) {
      tbase[u] = smraw + off + slot * 8;
      off += (size_t)ch.nk[u] * 128;
      mp[u] = imaps + (size_t)(ch.unit0 + u) * nRB * 256 + slot * 16;
    }
  }
  for (int64_t st = s0 + warp; st < s1; st += RB_W) {
    const int64_t r0 = st * LMM_STEP + half * 32;
    uint4 m[NU][2];
#pragma unroll
    for (int u = 0; u < NU; u++) {
      const uint8_t* src = mp[u] + (r0 >> 4) * 256;
      m[u][0] = __ldg((const uint4*)src);
      m[u][1] = __ldg((const uint4*)(src + 256));
    }
#pragma unroll
    for (int sub = 0; sub < 2; sub++) {
      double acc[16];
#pragma unroll
      for (int i = 0; i < 16; i++) acc[i] = 0.0;
#pragma unroll
      for (int u = 0; u < NU; u++) {
        const uint4 w = m[u][sub];
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        const unsigned char* T = tbase[u];
#pragma unroll
        for (int i = 0; i < 16; i++) acc[i] += *(const double*)(T + byte_x128(ww[i >> 2], i & 3));
      }
      // reduce-scatter over the half-warp: after the stage with distance d, a lane keeps the rows whose bit d
      // equals its own slot bit
#pragma unroll
      for (int d = 8; d >= 1; d >>= 1) {
        const bool up = (slot & d) != 0;
#pragma unroll
        for (int i = 0; i < d; i++) {
          const double lo = acc[i], hi = acc[i + d];
          const double recv = __shfl_xor_sync(0xffffffffu, up ? lo : hi, d);
          acc[i] = (up ? hi : lo) + recv;
        }
      }
      const int64_t row = r0 + sub * 16 + slot;
      if (row < nRows) out[row] = first ? acc[0] + init : out[row] + acc[0];
    }
  }
}

__global__ void __launch_bounds__(RB_W * 32, 1)
k_rmm_vec_b(const LmmChunk* __restrict__ chunks, int nChunks, const uint8_t* __restrict__ imaps, int64_t nRB,
            const double* __restrict__ P, int nRows, const double* __restrict__ constRow, double* __restrict__ out,
            int32_t* err) {
  extern __shared__ __align__(128) unsigned char smraw[];
  __shared__ __align__(8) uint64_t mbar;
  __shared__ LmmChunk ch;
  const int64_t nSteps = ((int64_t)nRows + LMM_STEP - 1) / LMM_STEP;
  const int64_t s0 = nSteps * blockIdx.x / gridDim.x, s1 = nSteps * (blockIdx.x + 1) / gridDim.x;
  const double init = constRow ? constRow[0] : 0.0;
  tma_barrier_init(&mbar);
  for (int c = 0; c < nChunks; c++) {
    __syncthreads();  // everyone is done with the previous chunk's tables and with `ch`
    if (threadIdx.x == 0) ch = chunks[c];
    __syncthreads();
    if (!tma_reload(smraw, P + ch.tblOff, (uint32_t)ch.tblDoubles * 8u, &mbar, (uint32_t)(c & 1))) {
      if (threadIdx.x == 0) atomicExch(err, 102);
      return;
    }
#define RB_CASE(N) case N: rmm_b_chunk<N>(ch, imaps, nRB, s0, s1, nRows, init, c == 0, out, smraw); break;
    switch (ch.nUnits) {
      RB_CASE(1) RB_CASE(2) RB_CASE(3) RB_CASE(4) RB_CASE(5) RB_CASE(6)
      default: rmm_b_chunk<7>(ch, imaps, nRB, s0, s1, nRows, init, c == 0, out, smraw); break;
    }
#undef RB_CASE
  }
}

// --------------------------------------------------------------------------------------------------
// RMM with two groups per dictionary read. When dictionaries are small, two groups g and h share one column
// slot: the slot's table holds P_g[a] + P_h[b] at entry (a << sh) | b (at most 256 entries), so one 8-byte read
// serves two cells -- the lookup bound of 16 reads per clock per SM then allows 32 cells per clock. The maps stay
// as registered; the kernel reads both groups' ids ([slab16][16-row block][a | b][slot][16 ids], one 128-bit load
// each) and combines them with one multiply-add per four rows. Otherwise identical to k_rmm_vec_b.
// --------------------------------------------------------------------------------------------------
__global__ void k_rmm_f_tables(const DevGroup* __restrict__ groups, const LmmChunk* __restrict__ chunks,
                               const FusedUnit* __restrict__ units, const double* __restrict__ v,
                               double* __restrict__ P) {
  const LmmChunk ch = chunks[blockIdx.x];
  int base = 0;
  for (int q = 0; q < ch.nUnits; q++) {
    const int n = ch.nk[q] * 16;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < n; e += gridDim.y * blockDim.x) {  // gridDim.y CTAs per chunk
      const FusedUnit u = units[(ch.unit0 + q) * 16 + (e & 15)];
      const int k = e >> 4;
      double val = 0.0;
      if (u.ga >= 0) {
        const int a = k >> u.sh, b = k & ((1 << u.sh) - 1);
        if (a < u.nva && (u.gb < 0 ? b == 0 : b < u.nvb)) {
          const DevGroup& ga = groups[u.ga];
          for (int h = 0; h < ga.gCols; h++) val += ga.dict[(size_t)a * ga.gCols + h] * v[ga.cols[h]];
          if (u.gb >= 0) {
            const DevGroup& gb = groups[u.gb];
            double vb = 0.0;
            for (int h = 0; h < gb.gCols; h++) vb += gb.dict[(size_t)b * gb.gCols + h] * v[gb.cols[h]];
            val += vb;
          }
        }
      }
      P[ch.tblOff + base + e] = val;
    }
    base += n;
  }
}

template <int NU>
__device__ __forceinline__ void rmm_f_chunk(const LmmChunk& ch, const FusedUnit* __restrict__ units,
                                            const uint8_t* __restrict__ fmaps, int64_t nRB, int64_t s0, int64_t s1,
                                            int nRows, double init, bool first, double* __restrict__ out,
                                            const unsigned char* smraw) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slot = lane & 15, half = lane >> 4;
  const unsigned char* tbase[NU];
  const uint8_t* mp[NU];
  uint32_t mul[NU];  // 1 << sh of this lane's slot
  {
    size_t off = 0;
#pragma unroll
    for (int u = 0; u < NU; u++) {
      tbase[u] = smraw + off + slot * 8;
      off += (size_t)ch.nk[u] * 128;
      mp[u] = fmaps + (size_t)(ch.unit0 + u) * nRB * 512 + slot * 16;
      mul[u] = 1u << units[(ch.unit0 + u) * 16 + slot].sh;
    }
  }
  // The ids of the next 16 rows are loaded before the current 16 are looked up (two register buffers): with a few
  // steps per warp on a short matrix, waiting for each load before issuing the next was most of the run time.
  auto load_ids = [&](int64_t st, int sub, uint4 (&ma)[NU], uint4 (&mb)[NU]) {
    const int64_t rb = ((st * LMM_STEP + half * 32) >> 4) + sub;
#pragma unroll
    for (int u = 0; u < NU; u++) {
      const uint8_t* src = mp[u] + rb * 512;
      ma[u] = __ldg((const uint4*)src);          // 16 lanes x 16 bytes: two full 128-byte lines per half-warp
      mb[u] = __ldg((const uint4*)(src + 256));
    }
  };
  auto lookup_rows = [&](int64_t st, int sub, const uint4 (&ma)[NU], const uint4 (&mb)[NU]) {
    double acc[16];
#pragma unroll
    for (int i = 0; i < 16; i++) acc[i] = 0.0;
#pragma unroll
    for (int u = 0; u < NU; u++) {
      // ids stay below 256 after the shift, so the four bytes of a word never carry into each other
      const uint32_t ww[4] = {ma[u].x * mul[u] + mb[u].x, ma[u].y * mul[u] + mb[u].y, ma[u].z * mul[u] + mb[u].z,
                              ma[u].w * mul[u] + mb[u].w};
      const unsigned char* T = tbase[u];
#pragma unroll
      for (int i = 0; i < 16; i++) acc[i] += *(const double*)(T + byte_x128(ww[i >> 2], i & 3));
    }
#pragma unroll
    for (int d = 8; d >= 1; d >>= 1) {
      const bool up = (slot & d) != 0;
#pragma unroll
      for (int i = 0; i < d; i++) {
        const double lo = acc[i], hi = acc[i + d];
        const double recv = __shfl_xor_sync(0xffffffffu, up ? lo : hi, d);
        acc[i] = (up ? hi : lo) + recv;
      }
    }
    const int64_t row = st * LMM_STEP + half * 32 + sub * 16 + slot;
    if (row < nRows) out[row] = first ? acc[0] + init : out[row] + acc[0];
  };
  uint4 a0[NU], b0[NU], a1[NU], b1[NU];
  int64_t st = s0 + warp;
  if (st < s1) load_ids(st, 0, a0, b0);
  for (; st < s1; st += LMM_W) {
    load_ids(st, 1, a1, b1);
    lookup_rows(st, 0, a0, b0);
    if (st + LMM_W < s1) load_ids(st + LMM_W, 0, a0, b0);
    lookup_rows(st, 1, a1, b1);
  }
}

__global__ void __launch_bounds__(LMM_T, 1)
k_rmm_vec_f(const LmmChunk* __restrict__ chunks, int nChunks, const FusedUnit* __restrict__ units,
            const uint8_t* __restrict__ fmaps, int64_t nRB, const double* __restrict__ P, int nRows,
            const double* __restrict__ constRow, double* __restrict__ out, int32_t* err) {
  extern __shared__ __align__(128) unsigned char smraw[];
  __shared__ __align__(8) uint64_t mbar;
  __shared__ LmmChunk ch;
  const int64_t nSteps = ((int64_t)nRows + LMM_STEP - 1) / LMM_STEP;
  const int64_t s0 = nSteps * blockIdx.x / gridDim.x, s1 = nSteps * (blockIdx.x + 1) / gridDim.x;
  const double init = constRow ? constRow[0] : 0.0;
  tma_barrier_init(&mbar);
  for (int c = 0; c < nChunks; c++) {
    __syncthreads();
    if (threadIdx.x == 0) ch = chunks[c];
    __syncthreads();
    if (!tma_reload(smraw, P + ch.tblOff, (uint32_t)ch.tblDoubles * 8u, &mbar, (uint32_t)(c & 1))) {
      if (threadIdx.x == 0) atomicExch(err, 103);
      return;
    }
    switch (ch.nUnits) {
      case 1: rmm_f_chunk<1>(ch, units, fmaps, nRB, s0, s1, nRows, init, c == 0, out, smraw); break;
      case 2: rmm_f_chunk<2>(ch, units, fmaps, nRB, s0, s1, nRows, init, c == 0, out, smraw); break;
      case 3: rmm_f_chunk<3>(ch, units, fmaps, nRB, s0, s1, nRows, init, c == 0, out, smraw); break;
      default: rmm_f_chunk<4>(ch, units, fmaps, nRB, s0, s1, nRows, init, c == 0, out, smraw); break;
    }
  }
}

// [slab16][16-row block][a | b][slot][16 ids]: a half-warp's load of the a ids (and of the b ids) is 256 contiguous bytes
__global__ void k_rmm_f_interleave(const uint8_t* const* __restrict__ mapA, const uint8_t* const* __restrict__ mapB,
                                   int nSlots, int nRows, int64_t nRB, uint8_t* __restrict__ out) {
  const int64_t total = (int64_t)nSlots * nRB * 2;
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
    const int slot = (int)(g & 15);
    const int which = (int)((g >> 4) & 1);
    const int64_t rb = (g >> 5) % nRB;
    const int64_t slab = (g >> 5) / nRB;
    const int unit = (int)slab * 16 + slot;
    const uint8_t* map = unit < nSlots ? (which ? mapB[unit] : mapA[unit]) : nullptr;
    uint4 v = make_uint4(0, 0, 0, 0);
    const int64_t r = rb * 16;
    if (map && r < nRows) {
      if (r + 16 <= nRows) v = *(const uint4*)(map + r);
      else {
        __align__(16) uint8_t tmp[16];
        for (int i = 0; i < 16; i++) tmp[i] = (r + i < nRows) ? map[r + i] : 0;
        v = *(const uint4*)tmp;
      }
    }
    ((uint4*)out)[g] = v;
  }
}

// Device layout of the maps for k_lmm_vec_u8: [slab of 16 column slots][16-row block][slot][16 ids].
// A half-warp (one lane per slot) then reads 256 contiguous bytes per 128-bit load instead of 16 scattered
// lines. Built once at plan time; unused slots and rows past the end hold id 0.
__global__ void k_lmm_interleave(const uint8_t* const* __restrict__ slotMap, int nSlots, int nUnits, int nRows,
                                 int64_t nRB, uint8_t* __restrict__ out) {
  const int64_t total = (int64_t)nSlots * nRB;
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
    const int slot = (int)(g & 15);
    const int64_t rb = (g >> 4) % nRB;
    const int64_t slab = (g >> 4) / nRB;
    const int unit = (int)slab * 16 + slot;
    uint4 v = make_uint4(0, 0, 0, 0);
    const int64_t r = rb * 16;
    if (unit < nUnits && r < nRows) {
      const uint8_t* src = slotMap[unit] + r;
      if (r + 16 <= nRows) v = *(const uint4*)src;
      else {
        __align__(16) uint8_t tmp[16];
        for (int i = 0; i < 16; i++) tmp[i] = (r + i < nRows) ? src[i] : 0;
        v = *(const uint4*)tmp;
      }
    }
    ((uint4*)out)[g] = v;
  }
}

// bit map -> byte map (one id per byte), used once at plan time
__global__ void k_bits_to_bytes(const unsigned long long* __restrict__ bits, uint8_t* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = (uint8_t)((bits[i >> 6] >> (i & 63)) & 1ULL);
}

// --------------------------------------------------------------------------------------------------
// plan
// --------------------------------------------------------------------------------------------------
template <typename T>
static int64_t plan_upload(FastPlan* fp, const std::vector<T>& h, T** d) {
  *d = nullptr;
  if (h.empty()) return CLA_OK;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, h.size() * sizeof(T));
  if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc plan: ") + cudaGetErrorString(e));
  fp->allocs.push_back(p);
  CLA_CUDA(cudaMemcpy(p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
  *d = (T*)p;
  return CLA_OK;
}

void fast_plan_free(Matrix* m) {
  if (!m->fast) return;
  for (void* p : m->fast->allocs) cudaFree(p);
  delete m->fast;
  m->fast = nullptr;
}

int64_t fast_plan_build(Matrix* m) {
  FastPlan* fp = new FastPlan();
  m->fast = fp;
  if (m->nRows < FAST_MIN_ROWS || m->nDev == 0) return CLA_OK;
  // the groups these kernels cover: dense maps, at most 256 tuples, one byte (or bit) per cell
  std::vector<DevGroup> G;
  std::vector<int> selIdx;
  for (int gi = 0; gi < m->nDev; gi++) {
    const DevGroup& g = m->groups[gi];
    if (g.type != GT_DDC || g.nVals > 256 || g.nVals < 1) continue;
    if (g.mapType != CLA_MAP_UBYTE && g.mapType != CLA_MAP_BYTE && g.mapType != CLA_MAP_BIT) continue;
    G.push_back(g);
    selIdx.push_back(gi);
  }
  const bool all = (int)G.size() == m->nDev;
  int nUnitsSel = 0;
  for (auto& g : G) nUnitsSel += g.gCols;
  if (G.empty() || (!all && nUnitsSel < 16)) return CLA_OK;  // too few columns to be worth a separate pass
  fp->partial = !all;
  const int nG = (int)G.size();
  fp->nG = nG;
  int64_t rc;
  // byte maps for every group (bit maps are expanded once)
  std::vector<const uint8_t*> gmap(nG);
  for (int gi = 0; gi < nG; gi++) {
    const DevGroup& g = G[gi];
    if (g.mapType == CLA_MAP_BIT) {
      void* p = nullptr;
      CLA_CUDA(cudaMalloc(&p, (size_t)m->nRows + 64));
      fp->allocs.push_back(p);
      m->deviceBytes += m->nRows;
      k_bits_to_bytes<<<std::min(4096, (m->nRows + 255) / 256), 256, 0, m->stream>>>((const unsigned long long*)g.map,
                                                                                   (uint8_t*)p, m->nRows);
      gmap[gi] = (const uint8_t*)p;
    } else
      gmap[gi] = (const uint8_t*)g.map;
  }
  CLA_CUDA(cudaStreamSynchronize(m->stream));

  // ---- RMM: groups ordered by table size so the small (conflict-free) tables pack together ----
  std::vector<int> order(nG);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return G[a].nVals < G[b].nVals; });
  int64_t total = 0;
  for (int gi : order) total += (G[gi].nVals + 1) & ~1;
  const int budget = total * 8 <= 40 * 1024 ? 40 * 1024 : 96 * 1024;  // small: many CTAs per SM; else two per SM
  std::vector<const uint8_t*> maps(nG);
  std::vector<int> tblOff(nG), groupOf(nG);
  std::vector<int64_t> imgOff(nG);
  int64_t img = 0;
  RmmChunk cur{0, 0, 0, 0};
  for (int i = 0; i < nG; i++) {
    const int gi = order[i];
    const int pad = (G[gi].nVals + 1) & ~1;
    const int perGroup = 8 + 4;  // map pointer + offset kept in shared memory
    if (cur.g1 > cur.g0 && (cur.tblDoubles + pad) * 8 + (cur.g1 - cur.g0 + 1) * perGroup > budget) {
      fp->rchunks.push_back(cur);
      cur = RmmChunk{i, i, 0, img};
    }
    maps[i] = gmap[gi];
    groupOf[i] = selIdx[gi];
    tblOff[i] = cur.tblDoubles;
    imgOff[i] = img;
    cur.tblDoubles += pad;
    cur.g1 = i + 1;
    img += pad;
  }
  fp->rchunks.push_back(cur);
  fp->pImgDoubles = img;
  if ((rc = plan_upload(fp, maps, &fp->dMaps)) < 0) return rc;
  if ((rc = plan_upload(fp, tblOff, &fp->dTblOff)) < 0) return rc;
  if ((rc = plan_upload(fp, groupOf, &fp->dGroupOf)) < 0) return rc;
  if ((rc = plan_upload(fp, imgOff, &fp->dImgOff)) < 0) return rc;

  // ---- LMM: one column slot per (group, column), in output-column order; 16 slots per unit ----
  // (A chunk holds at most LMM_MAX_UNITS units and their tables fit at any depth, so nothing is gained by packing
  // shallow tables together; in column order the 16 slots of a unit are neighbours in a decompressed row.)
  struct Unit { int g, j, nv, col; };
  std::vector<Unit> units;
  for (int gi = 0; gi < nG; gi++) {
    std::vector<int32_t> cols(G[gi].gCols);
    CLA_CUDA(cudaMemcpy(cols.data(), G[gi].cols, cols.size() * 4, cudaMemcpyDeviceToHost));
    for (int j = 0; j < G[gi].gCols; j++) units.push_back({gi, j, G[gi].nVals, cols[j]});
  }
  std::stable_sort(units.begin(), units.end(), [](const Unit& a, const Unit& b) { return a.col < b.col; });
  fp->nUnits = (int)units.size();
  const int nU16 = (fp->nUnits + 15) / 16;
  fp->nSlots = nU16 * 16;
  // unused slots of the last unit read the map of the last column (its ids stay inside the unit's table depth)
  std::vector<const uint8_t*> slotMap(fp->nSlots, gmap[units.back().g]);
  std::vector<int> slotCol(fp->nSlots, -1);
  std::vector<int> unitNk(nU16, 1);
  // host copies of the dictionaries
  std::vector<std::vector<double>> dicts(nG);
  for (int gi = 0; gi < nG; gi++) {
    dicts[gi].resize((size_t)G[gi].nVals * G[gi].gCols);
    CLA_CUDA(cudaMemcpy(dicts[gi].data(), G[gi].dict, dicts[gi].size() * 8, cudaMemcpyDeviceToHost));
  }
  for (int u = 0; u < fp->nUnits; u++) unitNk[u / 16] = std::max(unitNk[u / 16], units[u].nv);
  // chunks: greedily pack units up to the shared-memory budget and LMM_MAX_UNITS
  const size_t redBytes = (size_t)LMM_W * LMM_PART * 8;
  const size_t lmmBudget = SMEM_MAX - 2048;
  std::vector<double> image;
  LmmChunk lc{};
  lc.unit0 = 0;
  auto flush = [&]() {
    lc.tblDoubles = 0;
    for (int q = 0; q < lc.nUnits; q++) lc.tblDoubles += lc.nk[q] * 16;
    lc.tblOff = (int64_t)image.size();
    image.resize(image.size() + lc.tblDoubles, 0.0);
    size_t off = lc.tblOff;
    for (int q = 0; q < lc.nUnits; q++) {
      for (int s = 0; s < 16; s++) {
        const int u = (lc.unit0 + q) * 16 + s;
        if (u >= fp->nUnits) continue;
        const Unit& un = units[u];
        const int gc = G[un.g].gCols;
        for (int k = 0; k < un.nv; k++) image[off + (size_t)k * 16 + s] = dicts[un.g][(size_t)k * gc + un.j];
      }
      off += (size_t)lc.nk[q] * 16;
    }
    fp->lchunks.push_back(lc);
  };
  size_t curBytes = 0;
  lc.nUnits = 0;
  for (int q = 0; q < nU16; q++) {
    const size_t b = (size_t)unitNk[q] * 128;
    if (lc.nUnits == LMM_MAX_UNITS || (lc.nUnits > 0 && std::max(curBytes + b, redBytes) > lmmBudget)) {
      flush();
      lc = LmmChunk{};
      lc.unit0 = q;
      lc.nUnits = 0;
      curBytes = 0;
    }
    lc.nk[lc.nUnits++] = unitNk[q];
    curBytes += b;
  }
  flush();
  for (int u = 0; u < fp->nUnits; u++) {
    slotMap[u] = gmap[units[u].g];
    slotCol[u] = units[u].col;
  }
  // CTAs per chunk in proportion to its cost, one CTA per SM in total. Cost per 64-row warp step in
  // L1 data-pipe wavefronts: 64 per unit for the dictionary reads, 8 per unit for the map loads and
  // 64 for the left vector (which does not depend on the number of units).
  const int totalCta = std::max(m->smCount, (int)fp->lchunks.size());
  double totalCost = 0;
  auto chunkCost = [](const LmmChunk& c) { return 72.0 * c.nUnits + 64.0; };
  for (auto& c : fp->lchunks) totalCost += chunkCost(c);
  int cta = 0;
  const int64_t nSteps = ((int64_t)m->nRows + LMM_STEP - 1) / LMM_STEP;
  std::vector<int> share(fp->lchunks.size());
  int used = 0;
  for (size_t i = 0; i < fp->lchunks.size(); i++) {
    share[i] = std::max(1, (int)(totalCta * chunkCost(fp->lchunks[i]) / totalCost));
    used += share[i];
  }
  for (size_t i = 0; used < totalCta; i = (i + 1) % fp->lchunks.size(), used++) share[i]++;  // hand out the remainder
  for (size_t i = 0; i < fp->lchunks.size(); i++) {
    auto& c = fp->lchunks[i];
    const int n = (int)std::min<int64_t>(share[i], nSteps);
    c.cta0 = cta;
    c.nCta = n;
    cta += n;
  }
  fp->lmmGrid = cta;
  if ((rc = plan_upload(fp, fp->lchunks, &fp->dLChunks)) < 0) return rc;
  if ((rc = plan_upload(fp, slotMap, &fp->dSlotMap)) < 0) return rc;
  if ((rc = plan_upload(fp, slotCol, &fp->dSlotCol)) < 0) return rc;
  {
    fp->nRB = (((int64_t)m->nRows + LMM_STEP - 1) / LMM_STEP) * (LMM_STEP / 16);
    const size_t bytes = (size_t)fp->nSlots * fp->nRB * 16;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc interleaved maps: ") + cudaGetErrorString(e));
    fp->allocs.push_back(p);
    fp->dLmmMaps = (uint8_t*)p;
    m->deviceBytes += (int64_t)bytes;
    k_lmm_interleave<<<m->smCount * 8, 256, 0, m->stream>>>(fp->dSlotMap, fp->nSlots, fp->nUnits, m->nRows, fp->nRB,
                                                           fp->dLmmMaps);
    CLA_CUDA(cudaStreamSynchronize(m->stream));
  }
  if ((rc = plan_upload(fp, image, &fp->dLmmTables)) < 0) return rc;
  fp->imageDoubles = image.size();
  for (auto& g : G) fp->maxNVals = std::max(fp->maxNVals, g.nVals);
  m->deviceBytes += (int64_t)image.size() * 8;
  CLA_CUDA(cudaFuncSetAttribute(k_lmm_vec_u8, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX - 1024));
  CLA_CUDA(cudaFuncSetAttribute(k_rmm_vec_b, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX - 1024));
  CLA_CUDA(cudaFuncSetAttribute(k_decomp_fast, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX - 2048));
  CLA_CUDA(cudaFuncSetAttribute(k_rmm_vec_u8<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
  CLA_CUDA(cudaFuncSetAttribute(k_rmm_vec_u8<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
  CLA_CUDA(cudaFuncSetAttribute(k_rmm_vec_u8<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
  // ---- RMM with two groups per lookup, when at least half of the groups find a partner ----
  {
    std::vector<int> byNv(nG);
    std::iota(byNv.begin(), byNv.end(), 0);
    std::stable_sort(byNv.begin(), byNv.end(), [&](int a, int b) { return G[a].nVals < G[b].nVals; });
    auto bitsFor = [](int nv) { int sh = 0; while ((1 << sh) < nv) sh++; return sh; };
    std::vector<FusedUnit> fu;
    int lo = 0, hi = nG - 1, paired = 0;
    while (lo <= hi) {  // the largest remaining dictionary takes the smallest remaining partner that still fits
      const int a = byNv[hi];
      if (lo < hi) {
        const int b = byNv[lo];
        const int sh = bitsFor(G[b].nVals);
        if ((G[a].nVals << sh) <= 256) {
          fu.push_back(FusedUnit{a, b, sh, G[a].nVals, G[b].nVals});
          paired += 2;
          lo++;
          hi--;
          continue;
        }
      }
      fu.push_back(FusedUnit{a, -1, 0, G[a].nVals, 1});
      hi--;
    }
    // (fast_rmm_vec takes this kernel below 4M rows only: no second copy of the maps for taller matrices)
    if (paired * 2 >= nG && !fp->partial && m->nRows < (4 << 20)) {
      std::stable_sort(fu.begin(), fu.end(), [](const FusedUnit& x, const FusedUnit& y) { return (x.nva << x.sh) > (y.nva << y.sh); });
      fp->nFused = (int)fu.size();
      const int nU16F = (fp->nFused + 15) / 16;
      const int nSlotsF = nU16F * 16;
      std::vector<const uint8_t*> mapA(nSlotsF, nullptr), mapB(nSlotsF, nullptr);
      std::vector<FusedUnit> units(nSlotsF, FusedUnit{-1, -1, 0, 1, 1});
      std::vector<int> nk(nU16F, 1);
      for (int u = 0; u < fp->nFused; u++) {
        mapA[u] = gmap[fu[u].ga];
        mapB[u] = fu[u].gb >= 0 ? gmap[fu[u].gb] : nullptr;
        units[u] = FusedUnit{selIdx[fu[u].ga], fu[u].gb >= 0 ? selIdx[fu[u].gb] : -1, fu[u].sh, fu[u].nva, fu[u].nvb};
        nk[u / 16] = std::max(nk[u / 16], fu[u].nva << fu[u].sh);
      }
      LmmChunk fc{};
      int64_t img = 0;
      size_t cur = 0;
      auto flushF = [&]() {
        fc.tblDoubles = 0;
        for (int q = 0; q < fc.nUnits; q++) fc.tblDoubles += fc.nk[q] * 16;
        fc.tblOff = img;
        img += fc.tblDoubles;
        fp->fchunks.push_back(fc);
      };
      fc.unit0 = 0;
      fc.nUnits = 0;
      for (int q = 0; q < nU16F; q++) {
        const size_t b = (size_t)nk[q] * 128;
        if (fc.nUnits == 4 || (fc.nUnits > 0 && cur + b > (size_t)SMEM_MAX - 2048)) {
          flushF();
          fc = LmmChunk{};
          fc.unit0 = q;
          fc.nUnits = 0;
          cur = 0;
        }
        fc.nk[fc.nUnits++] = nk[q];
        cur += b;
      }
      flushF();
      fp->fImageDoubles = (size_t)img;
      const uint8_t** dA = nullptr;
      const uint8_t** dB = nullptr;
      if ((rc = plan_upload(fp, mapA, &dA)) < 0) return rc;
      if ((rc = plan_upload(fp, mapB, &dB)) < 0) return rc;
      if ((rc = plan_upload(fp, units, &fp->dFUnits)) < 0) return rc;
      if ((rc = plan_upload(fp, fp->fchunks, &fp->dFChunks)) < 0) return rc;
      const size_t bytes = (size_t)nSlotsF * fp->nRB * 32;
      void* pm = nullptr;
      cudaError_t e = cudaMalloc(&pm, bytes);
      if (e != cudaSuccess) return fail(CLA_ERR_NOMEM, std::string("cudaMalloc fused maps: ") + cudaGetErrorString(e));
      fp->allocs.push_back(pm);
      fp->dFMaps = (uint8_t*)pm;
      m->deviceBytes += (int64_t)bytes;
      k_rmm_f_interleave<<<m->smCount * 8, 256, 0, m->stream>>>(dA, dB, nSlotsF, m->nRows, fp->nRB, fp->dFMaps);
      CLA_CUDA(cudaStreamSynchronize(m->stream));
      CLA_CUDA(cudaFuncSetAttribute(k_rmm_vec_f, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX - 1024));
      fp->fusedOk = true;
    }
  }
  if (fp->partial) {  // tell the general kernels which groups are taken care of
    for (int gi : selIdx) m->groups[gi].inFast = 1;
    CLA_CUDA(cudaMemcpy(m->dGroups, m->groups.data(), sizeof(DevGroup) * m->groups.size(), cudaMemcpyHostToDevice));
  }
  fp->ok = true;
  return CLA_OK;
}

// --------------------------------------------------------------------------------------------------
// launchers
// --------------------------------------------------------------------------------------------------
__global__ void k_const_dot(const double* __restrict__ constV, const double* __restrict__ v, int n, double* out) {
  double s = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += constV[i] * v[i];
  __shared__ double sh[256];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int d = 128; d; d >>= 1) {
    if ((int)threadIdx.x < d) sh[threadIdx.x] += sh[threadIdx.x + d];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = sh[0];
}

static int64_t fast_rmm_vec_b(Matrix* m, FastPlan* fp, const double* dV, double* dOut, cudaStream_t s) {
  int64_t rc;
  const size_t pBytes = ((size_t)fp->imageDoubles * 8 + 255) & ~(size_t)255;
  if ((rc = ensure_scratch(m, pBytes + 256)) < 0) return rc;
  double* P = (double*)m->scratch;
  double* constRow = nullptr;
  k_rmm_b_tables<<<dim3((unsigned)fp->lchunks.size(), 16), 256, 0, s>>>(fp->dLChunks, fp->dSlotCol, fp->dLmmTables, dV, P);
  m->stats.kernel_launches++;
  if (m->hasConst) {
    constRow = (double*)((char*)m->scratch + pBytes);
    k_const_dot<<<1, 256, 0, s>>>(m->dConstV, dV, m->nCols, constRow);
    m->stats.kernel_launches++;
  }
  size_t smem = 1024;
  for (auto& c : fp->lchunks) smem = std::max(smem, (size_t)c.tblDoubles * 8);
  const int64_t nSteps = ((int64_t)m->nRows + LMM_STEP - 1) / LMM_STEP;
  const int grid = (int)std::min<int64_t>(m->smCount, nSteps);
  prof_begin(m, s);
  k_rmm_vec_b<<<grid, RB_W * 32, smem, s>>>(fp->dLChunks, (int)fp->lchunks.size(), fp->dLmmMaps, fp->nRB, P, m->nRows, constRow,
                                        dOut, m->dErr);
  prof_end(m, s);
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return fp->partial ? 2 : 1;
}

static int64_t fast_rmm_vec_f(Matrix* m, FastPlan* fp, const double* dV, double* dOut, cudaStream_t s) {
  int64_t rc;
  const size_t pBytes = ((size_t)fp->fImageDoubles * 8 + 255) & ~(size_t)255;
  if ((rc = ensure_scratch(m, pBytes + 256)) < 0) return rc;
  double* P = (double*)m->scratch;
  double* constRow = nullptr;
  k_rmm_f_tables<<<dim3((unsigned)fp->fchunks.size(), 16), 256, 0, s>>>(m->dGroups, fp->dFChunks, fp->dFUnits, dV, P);
  m->stats.kernel_launches++;
  if (m->hasConst) {
    constRow = (double*)((char*)m->scratch + pBytes);
    k_const_dot<<<1, 256, 0, s>>>(m->dConstV, dV, m->nCols, constRow);
    m->stats.kernel_launches++;
  }
  size_t smem = 1024;
  for (auto& c : fp->fchunks) smem = std::max(smem, (size_t)c.tblDoubles * 8);
  const int64_t nSteps = ((int64_t)m->nRows + LMM_STEP - 1) / LMM_STEP;
  const int grid = (int)std::min<int64_t>(m->smCount, nSteps);
  prof_begin(m, s);
  k_rmm_vec_f<<<grid, LMM_T, smem, s>>>(fp->dFChunks, (int)fp->fchunks.size(), fp->dFUnits, fp->dFMaps, fp->nRB, P, m->nRows,
                                        constRow, dOut, m->dErr);
  prof_end(m, s);
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return 1;
}

bool fast_plan_ok(const Matrix* m) { return m->fast && m->fast->ok; }
bool fast_plan_partial(const Matrix* m) { return m->fast && m->fast->ok && m->fast->partial; }

// Rows [r0, r1) of the decompressed matrix into dOut (row r0 first) when every column is a slot of the plan and no
// column belongs to two groups; 0 = not covered (the caller takes the tile kernel).
int64_t fast_decompress(Matrix* m, int r0, int r1, double* dOut, cudaStream_t s) {
  FastPlan* fp = m->fast;
  if (!fp || !fp->ok || fp->partial || !fp->dLmmMaps || !m->colSrcValid || fp->nUnits != m->nCols || (r0 % LMM_STEP)) return 0;
  static const bool off = getenv("CLA_DECOMP_TILES") != nullptr;
  if (off) return 0;
  size_t smem = 0;
  for (auto& c : fp->lchunks) smem = std::max(smem, (size_t)c.tblDoubles * 8);
  k_decomp_fast<<<fp->lmmGrid, DEC_T, smem, s>>>(fp->dLChunks, (int)fp->lchunks.size(), fp->dLmmMaps, fp->nRB, fp->dLmmTables,
                                                fp->dSlotCol, m->hasConst ? m->dConstV : nullptr, dOut, m->nCols, r0, r1,
                                                m->dErr);
  m->stats.kernel_launches++;
  CLA_CUDA(cudaGetLastError());
  return 1;
}

int64_t fast_rmm_vec(Matrix* m, const double* dV, double* dOut, cudaStream_t s) {
  FastPlan* fp = m->fast;
  if (!fp || !fp->ok || ((uintptr_t)dOut & 15)) return 0;  // 128-bit stores need an aligned output
  // Two groups per lookup pays off on short matrices, where the row-per-thread kernel cannot keep enough loads
  // in flight (measured: 1M rows 46.6 vs 52.5 us); on tall ones the second map load and the shuffles cost more
  // than the saved reads (10M rows: 344 vs 326 us).
  if (fp->fusedOk && m->nRows < (4 << 20) && !getenv("CLA_NO_FUSED_RMM")) return fast_rmm_vec_f(m, fp, dV, dOut, s);
  if (fp->maxNVals > 16) return fast_rmm_vec_b(m, fp, dV, dOut, s);  // deep tables: the conflict-free layout
  int64_t rc;
  const size_t pBytes = ((size_t)fp->pImgDoubles * 8 + 255) & ~(size_t)255;
  if ((rc = ensure_scratch(m, pBytes + 256)) < 0) return rc;
  double* P = (double*)m->scratch;
  double* constRow = nullptr;
  k_fast_ptable<<<fp->nG, 128, 0, s>>>(m->dGroups, fp->dGroupOf, fp->dImgOff, fp->nG, dV, P);
  m->stats.kernel_launches++;
  if (m->hasConst) {
    constRow = (double*)((char*)m->scratch + pBytes);
    k_const_dot<<<1, 256, 0, s>>>(m->dConstV, dV, m->nCols, constRow);
    m->stats.kernel_launches++;
  }
  // rows per thread: 128-bit map loads from about two million rows on, 32-bit ones below (measured on 100 groups of
  // 16 values, ms per product for 4 / 8 / 16 rows per thread: 1M rows 0.052 / 0.071 / 0.057, 3M rows 0.127 / 0.142 /
  // 0.127, 10M rows 0.358 / 0.449 / 0.322; eight rows per thread lose at every size)
  int R = m->nRows >= (2 << 20) - 200000 ? 16 : 4;
  if (const char* e = getenv("CLA_RMM_ROWS_PER_THREAD")) {  // tuning aid
    const int v = atoi(e);
    if (v == 4 || v == 8 || v == 16) R = v;
  }
  const int nTiles = (m->nRows + RMM_T * R - 1) / (RMM_T * R);
  for (size_t c = 0; c < fp->rchunks.size(); c++) {
    const RmmChunk& ch = fp->rchunks[c];
    const size_t smem = (size_t)ch.tblDoubles * 8 + (size_t)(ch.g1 - ch.g0) * 12 + 16;
    auto kern = R == 16 ? k_rmm_vec_u8<16> : (R == 8 ? k_rmm_vec_u8<8> : k_rmm_vec_u8<4>);
    // as many CTAs as are resident at once (registers and shared memory decide): the tile loop does the rest, and
    // no partial second wave is left over
    int perSm = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kern, RMM_T, smem) != cudaSuccess || perSm < 1) {
      cudaGetLastError();
      perSm = 1;
    }
    const int grid = std::min(nTiles, m->smCount * perSm);
    if (c == 0) prof_begin(m, s);
    kern<<<grid, RMM_T, smem, s>>>(fp->dMaps, fp->dTblOff, ch.g0, ch.g1, P + ch.tblOff, ch.tblDoubles, m->nRows, constRow,
                                   dOut, c > 0 ? 1 : 0, m->dErr);
    if (c + 1 == fp->rchunks.size()) prof_end(m, s);
    m->stats.kernel_launches++;
  }
  CLA_CUDA(cudaGetLastError());
  return fp->partial ? 2 : 1;
}

int64_t fast_lmm_vec(Matrix* m, const double* dY, double* dOut, cudaStream_t s) {
  FastPlan* fp = m->fast;
  if (!fp || !fp->ok || ((uintptr_t)dY & 15)) return 0;  // 128-bit loads of the left vector need alignment
  int64_t rc;
  const size_t partBytes = (size_t)fp->lmmGrid * LMM_PART * 8;
  if ((rc = ensure_scratch(m, partBytes + 256)) < 0) return rc;
  double* partial = (double*)m->scratch;
  CLA_CUDA(cudaMemsetAsync(dOut, 0, sizeof(double) * (size_t)m->nCols, s));
  size_t smem = (size_t)LMM_W * LMM_PART * 8;
  for (auto& c : fp->lchunks) smem = std::max(smem, (size_t)c.tblDoubles * 8);
  prof_begin(m, s);
  const int64_t nSteps = ((int64_t)m->nRows + LMM_STEP - 1) / LMM_STEP;
  k_lmm_vec_u8<<<fp->lmmGrid, LMM_T, smem, s>>>(fp->dLChunks, (int)fp->lchunks.size(), fp->dLmmMaps, fp->nRB, fp->dLmmTables, dY,
                                               m->nRows, 0, nSteps, partial, m->dErr);
  prof_end(m, s);
  k_lmm_vec_final<<<dim3((unsigned)fp->lchunks.size(), LMM_MAX_UNITS), 512, 0, s>>>(fp->dLChunks, (int)fp->lchunks.size(), fp->dSlotCol,
                                                              partial, dOut, 1, fp->lmmGrid);
  m->stats.kernel_launches += 2;
  if (m->hasConst)
    if ((rc = launch_lmm_const(m, dY, 1, dOut, s)) < 0) return rc;
  CLA_CUDA(cudaGetLastError());
  return fp->partial ? 2 : 1;
}


// Q = 2 or 4 left rows (rows q of y at y + q * pitch, 16-byte aligned) in one pass; same return values as fast_lmm_vec.
template <int Q>
static int64_t fast_lmm_rows_t(Matrix* m, FastPlan* fp, const double* dY, size_t pitch, double* dOut, cudaStream_t s) {
  int64_t rc;
  const size_t partBytes = (size_t)fp->lmmGrid * Q * LMM_PART * 8;
  if ((rc = ensure_scratch(m, partBytes + 256)) < 0) return rc;
  double* partial = (double*)m->scratch;
  CLA_CUDA(cudaMemsetAsync(dOut, 0, sizeof(double) * (size_t)Q * m->nCols, s));
  size_t smem = (size_t)LQ_W * Q * LMM_PART * 8;
  for (auto& c : fp->lchunks) smem = std::max(smem, (size_t)c.tblDoubles * 8);
  static bool attr[64] = {};
  if (!attr[m->device & 63]) {
    CLA_CUDA(cudaFuncSetAttribute(k_lmm_vecq_u8<Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX - 1024));
    attr[m->device & 63] = true;
  }
  prof_begin(m, s);
  k_lmm_vecq_u8<Q><<<fp->lmmGrid, LQ_T, smem, s>>>(fp->dLChunks, (int)fp->lchunks.size(), fp->dLmmMaps, fp->nRB, fp->dLmmTables, dY,
                                                  pitch, m->nRows, partial, m->dErr);
  prof_end(m, s);
  k_lmm_vecq_final<<<dim3((unsigned)fp->lchunks.size(), LMM_MAX_UNITS, Q), 512, 0, s>>>(fp->dLChunks, (int)fp->lchunks.size(),
                                                                                       fp->dSlotCol, partial, dOut, Q, m->nCols);
  m->stats.kernel_launches += 2;
  if (m->hasConst)
    for (int q = 0; q < Q; q++)
      if ((rc = launch_lmm_const(m, dY + q * pitch, 1, dOut + (size_t)q * m->nCols, s)) < 0) return rc;
  CLA_CUDA(cudaGetLastError());
  return fp->partial ? 2 : 1;
}
int64_t fast_lmm_rows(Matrix* m, const double* dY, size_t pitch, int q, double* dOut, cudaStream_t s) {
  FastPlan* fp = m->fast;
  if (!fp || !fp->ok || ((uintptr_t)dY & 15) || (pitch & 1)) return 0;
  if (q == 4) return fast_lmm_rows_t<4>(m, fp, dY, pitch, dOut, s);
  if (q == 2) return fast_lmm_rows_t<2>(m, fp, dY, pitch, dOut, s);
  return fail(CLA_ERR_BAD_ARG, "fast_lmm_rows: 2 or 4 rows");
}

// Host-buffer t(y) %*% X with the upload of y overlapped with the product: y is copied in up to LMM_PIPE_MAX row ranges
// on a second stream, and the kernel for a range starts as soon as its slice has arrived. Returns 0 if the
// specialised kernel does not cover the matrix (the caller then copies y whole and takes the normal path).
constexpr int LMM_PIPE_MAX = 16;  // = the handle's copyDone events
static int lmm_pipe_depth() {
  static const int d = [] {
    const char* e = getenv("CLA_LMM_PIPE");
    const int v = e ? atoi(e) : 8;
    return v < 1 ? 1 : (v > LMM_PIPE_MAX ? LMM_PIPE_MAX : v);
  }();
  return d;
}
int64_t fast_lmm_vec_host(Matrix* m, const double* hostY, double* dY, double* dOut, cudaStream_t s) {
  FastPlan* fp = m->fast;
  if (!fp || !fp->ok || fp->partial || ((uintptr_t)dY & 15) || m->nRows < (1 << 20)) return 0;
  int64_t rc;
  const int LMM_PIPE = lmm_pipe_depth();
  const size_t partBytes = (size_t)LMM_PIPE * fp->lmmGrid * LMM_PART * 8;
  if ((rc = ensure_scratch(m, partBytes + 256)) < 0) return rc;
  if (!m->copyStream) {
    CLA_CUDA(cudaStreamCreateWithFlags(&m->copyStream, cudaStreamNonBlocking));
    for (int i = 0; i < LMM_PIPE_MAX; i++) CLA_CUDA(cudaEventCreateWithFlags(&m->copyDone[i], cudaEventDisableTiming));
  }
  double* partial = (double*)m->scratch;
  CLA_CUDA(cudaMemsetAsync(dOut, 0, sizeof(double) * (size_t)m->nCols, s));
  size_t smem = (size_t)LMM_W * LMM_PART * 8;
  for (auto& c : fp->lchunks) smem = std::max(smem, (size_t)c.tblDoubles * 8);
  const int64_t nSteps = ((int64_t)m->nRows + LMM_STEP - 1) / LMM_STEP;
  // the copy stream must not run ahead of work already queued on s that still reads dY
  CLA_CUDA(cudaEventRecord(m->ev1, s));
  CLA_CUDA(cudaStreamWaitEvent(m->copyStream, m->ev1, 0));
  // Row ranges of decreasing size (weights n, n - 1, ..., 1): the copy engine is the slower side, so every kernel has
  // finished before the next range has arrived, and what is left after the last byte has landed is the product over
  // the smallest range only.
  const int64_t wSum = (int64_t)LMM_PIPE * (LMM_PIPE + 1) / 2;
  auto range_start = [&](int i) { return nSteps * ((int64_t)i * (2 * LMM_PIPE - i + 1) / 2) / wSum; };  // i ranges: n + ... + (n - i + 1)
  auto range_rows = [&](int i, int64_t& sb, int64_t& se, int64_t& rb, int64_t& re) {
    sb = range_start(i), se = i + 1 == LMM_PIPE ? nSteps : range_start(i + 1);
    rb = sb * LMM_STEP, re = std::min<int64_t>(m->nRows, se * LMM_STEP);
  };
  // the kernel of row range i, once that range of y is on the copy stream
  auto launch_range = [&](int i) -> int64_t {
    int64_t sb, se, rb, re;
    range_rows(i, sb, se, rb, re);
    CLA_CUDA(cudaEventRecord(m->copyDone[i], m->copyStream));
    CLA_CUDA(cudaStreamWaitEvent(s, m->copyDone[i], 0));
    if (i == 0) prof_begin(m, s);
    k_lmm_vec_u8<<<fp->lmmGrid, LMM_T, smem, s>>>(fp->dLChunks, (int)fp->lchunks.size(), fp->dLmmMaps, fp->nRB, fp->dLmmTables,
                                                 dY, m->nRows, sb, se, partial + (size_t)i * fp->lmmGrid * LMM_PART,
                                                 m->dErr);
    if (i == LMM_PIPE - 1) prof_end(m, s);
    m->stats.kernel_launches++;
    return CLA_OK;
  };
  if (host_copy_staged(m, hostY, (size_t)m->nRows * 8)) {
    // y lives in pageable memory: host threads move it through the pinned ring, and every row range starts as soon
    // as its last slice is on the copy stream
    int nextRange = 0;
    rc = host_to_device_staged(m, dY, hostY, (size_t)m->nRows * 8, m->copyStream, [&](size_t bytesQueued) -> int64_t {
      while (nextRange < LMM_PIPE) {
        int64_t sb, se, rb, re;
        range_rows(nextRange, sb, se, rb, re);
        if ((size_t)re * 8 > bytesQueued) break;
        const int64_t r = launch_range(nextRange++);
        if (r < 0) return r;
      }
      return CLA_OK;
    });
    if (rc < 0) return rc;
    while (nextRange < LMM_PIPE)
      if ((rc = launch_range(nextRange++)) < 0) return rc;
  } else {
    for (int i = 0; i < LMM_PIPE; i++) {
      int64_t sb, se, rb, re;
      range_rows(i, sb, se, rb, re);
      if (re > rb) CLA_CUDA(cudaMemcpyAsync(dY + rb, hostY + rb, (size_t)(re - rb) * 8, cudaMemcpyHostToDevice, m->copyStream));
      if ((rc = launch_range(i)) < 0) return rc;
    }
  }
  k_lmm_vec_final<<<dim3((unsigned)fp->lchunks.size(), LMM_MAX_UNITS), 512, 0, s>>>(fp->dLChunks, (int)fp->lchunks.size(), fp->dSlotCol, partial,
                                                              dOut, LMM_PIPE, fp->lmmGrid);
  m->stats.kernel_launches++;
  if (m->hasConst)
    if ((rc = launch_lmm_const(m, dY, 1, dOut, s)) < 0) return rc;
  CLA_CUDA(cudaGetLastError());
  return 1;
}

// --------------------------------------------------------------------------------------------------
// t(y) %*% X without any device allocation.
//
// Some hosts may not allocate device memory when they call in: a runtime that has handed the whole GPU to
// its own memory pool (SystemDS's GPU memory manager works that way), or a service loop that must not hit
// cudaMalloc because the driver synchronises the device inside it. For them the per-CTA partial sums and the
// row sum of the left vector live in this fixed array instead of the handle's growable scratch. Every GPU
// whose context loads the library holds the array (about 450 KB) until the process exits.
// --------------------------------------------------------------------------------------------------
constexpr int NOALLOC_MAX_CTAS = 512;  // partial-sum rows available; one CTA per SM is launched, more only with > 148 column chunks
constexpr size_t NOALLOC_PARTIAL_DOUBLES = (size_t)NOALLOC_MAX_CTAS * LMM_PART;
static __device__ __align__(256) double g_noalloc_scratch[NOALLOC_PARTIAL_DOUBLES + 32];

static std::mutex g_noallocMu;
static double* g_noallocAddr[64] = {};  // device address of the array, per device ordinal

// The name g_noalloc_scratch is only a handle on the host; kernels need the address the device sees.
// Looked up once per device, with that device current.
static int64_t noalloc_address(int device, double** out) {
  if (device < 0 || device >= 64) return fail(CLA_ERR_BAD_ARG, "device ordinal out of range");
  std::lock_guard<std::mutex> lk(g_noallocMu);
  if (!g_noallocAddr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return fail(CLA_ERR_CUDA, std::string("cudaGetSymbolAddress(g_noalloc_scratch): ") + cudaGetErrorString(e));
    g_noallocAddr[device] = (double*)p;
  }
  *out = g_noallocAddr[device];
  return CLA_OK;
}

int64_t fast_lmm_vec_noalloc(Matrix* m, const double* dY, double* dOut, cudaStream_t s) {
  FastPlan* fp = m->fast;
  if (!fp || !fp->ok || fp->partial)
    return fail(CLA_ERR_UNSUPPORTED, "no-allocation product: needs dense-map groups with at most 256 tuples and byte maps");
  if ((uintptr_t)dY & 15) return fail(CLA_ERR_BAD_ARG, "no-allocation product: the left vector must be 16-byte aligned");
  if (fp->lmmGrid > NOALLOC_MAX_CTAS)
    return fail(CLA_ERR_UNSUPPORTED, "no-allocation product: the matrix needs " + std::to_string(fp->lmmGrid) +
                                         " partial-sum rows, the fixed scratch holds " + std::to_string(NOALLOC_MAX_CTAS));
  double* scratch = nullptr;
  int64_t rc = noalloc_address(m->device, &scratch);
  if (rc < 0) return rc;
  m->stats.calls_lmm++;
  double* partial = scratch;                           // fully rewritten by every launch
  double* rowSum = scratch + NOALLOC_PARTIAL_DOUBLES;  // accumulated with atomics: cleared below before use
  CLA_CUDA(cudaMemsetAsync(dOut, 0, sizeof(double) * (size_t)m->nCols, s));
  size_t smem = (size_t)LMM_W * LMM_PART * 8;
  for (auto& c : fp->lchunks) smem = std::max(smem, (size_t)c.tblDoubles * 8);
  const int64_t nSteps = ((int64_t)m->nRows + LMM_STEP - 1) / LMM_STEP;
  k_lmm_vec_u8<<<fp->lmmGrid, LMM_T, smem, s>>>(fp->dLChunks, (int)fp->lchunks.size(), fp->dLmmMaps, fp->nRB, fp->dLmmTables,
                                               dY, m->nRows, 0, nSteps, partial, m->dErr);
  k_lmm_vec_final<<<dim3((unsigned)fp->lchunks.size(), LMM_MAX_UNITS), 512, 0, s>>>(fp->dLChunks, (int)fp->lchunks.size(), fp->dSlotCol,
                                                              partial, dOut, 1, fp->lmmGrid);
  m->stats.kernel_launches += 2;
  if (m->hasConst)
    if ((rc = launch_lmm_const_with(m, dY, 1, dOut, rowSum, s)) < 0) return rc;
  CLA_CUDA(cudaGetLastError());
  return CLA_OK;
}

}  // namespace cla
