/*
 * CPU oracle for the SystemDS CLA matrix-multiply path -- TEST INFRASTRUCTURE ONLY (see cla_oracle.h).
 *
 * Every function cites the reference source it restates, by path inside the reference project:
 *   C/  = src/main/java/org/apache/sysds/runtime/compress/
 *   CG/ = C/colgroup/
 * Arithmetic follows the reference's summation structure (dictionary pre-aggregation, then
 * row-block decompress-and-sum for RMM; left pre-aggregation in 4 x 4 x 2048 blocks, then a
 * small preAgg x dictionary product for LMM; counts-scaled dictionary products for TSMM).
 * Thread decomposition follows the reference's task split and is realised with OpenMP.
 */
#include "cla_oracle.h"
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

const int BITMAP_BLOCK_SZ = 65535;  // C/CompressionSettings.java:46
const int BYTE_MAXV = 255;          // CG/offset/OffsetByte.java:34
const int CHAR_MAXV = 65535;        // CG/offset/OffsetChar.java:32

enum GType { G_DDC, G_SDC, G_RLE, G_OLE, G_UNC, G_CONST, G_EMPTY };

struct Map {
  int type = OCL_MAP_ZERO;
  int64_t size = 0;
  std::vector<uint64_t> bits;
  std::vector<uint8_t> b;
  std::vector<uint16_t> c;
  std::vector<int32_t> i;
  // CG/mapping/Map*.java getIndex: Bit :100, UByte :51, Byte :67, Char :68, CharPByte :67, Int :63
  inline int get(int64_t r) const {
    switch (type) {
      case OCL_MAP_ZERO: return 0;
      case OCL_MAP_BIT: return (int)((bits[r >> 6] >> (r & 63)) & 1ULL);
      case OCL_MAP_UBYTE: return (int)(int8_t)b[r];
      case OCL_MAP_BYTE: return b[r] & 0xFF;
      case OCL_MAP_CHAR: return c[r];
      case OCL_MAP_CHAR_BYTE: return (int)c[r] + ((int)b[r] << 16);
      default: return i[r];
    }
  }
};

struct Offset {
  int type = OCL_OFF_EMPTY;
  int first = 0, last = 0;
  std::vector<uint8_t> b;
  std::vector<uint16_t> c;
};

// Iterator with the semantics of CG/offset/AIterator.java: value(), getDataIndex(), next().
struct OffIter {
  const Offset& o;
  int row;
  int64_t index = 0;  // position in the delta array
  int64_t dataIndex = 0;
  bool valid;
  explicit OffIter(const Offset& off) : o(off), row(off.first), valid(off.type != OCL_OFF_EMPTY) {}
  inline bool atLast() const { return row == o.last; }
  // CG/offset/OffsetByte.java:201-213, OffsetChar.java:172-180, OffsetTwo: jumps to last
  inline void next() {
    if (o.type == OCL_OFF_BYTE) {
      uint8_t v = o.b[index];
      while (v == 0) { row += BYTE_MAXV; index++; v = o.b[index]; }
      row += v;
      index++;
    } else if (o.type == OCL_OFF_CHAR) {
      uint16_t v = o.c[index];
      while (v == 0) { row += CHAR_MAXV; index++; v = o.c[index]; }
      row += v;
      index++;
    } else {
      row = o.last;
    }
    dataIndex++;
  }
};

struct Group {
  GType type;
  std::vector<int> cols;
  int nVals = 0;
  std::vector<double> dict;  // [nVals x gCols] row-major, CG/dictionary/Dictionary.java:94-97
  Map map;
  Offset off;
  bool single = false;       // SDCSingle*: no map, one tuple
  std::vector<double> def;   // default tuple (empty => *Zeros)
  std::vector<int> ptr;      // RLE / OLE: CG/AColGroupOffset.java:39-55
  std::vector<uint16_t> data;
  std::vector<double> dense;  // UNC [nRows x gCols]
  int gCols() const { return (int)cols.size(); }
};

}  // namespace

struct ocl_matrix {
  int nRows, nCols;
  std::vector<Group> groups;
};

namespace {

/* ---------------------------------------------------------------------------------------------
 * Generic "visit every (row, tuple id)" walkers over a row range, one per index structure.
 * ------------------------------------------------------------------------------------------- */

// RLE skip: CG/ColGroupRLE.java:611-628 (skipScanVal) -- find first run of value k ending after rl.
template <class F>
void rle_walk(const Group& g, int k, int rl, int ru, F&& f) {
  // decode loop CG/ColGroupRLE.java:114-117: rs = re + data[p]; re = rs + data[p+1]
  int re = 0;
  for (int p = g.ptr[k]; p < g.ptr[k + 1]; p += 2) {
    int rs = re + g.data[p];
    re = rs + g.data[p + 1];
    if (re <= rl) continue;
    if (rs >= ru) break;
    int a = std::max(rs, rl), b = std::min(re, ru);
    f(a, b);
  }
}

// OLE segments: CG/ColGroupOLE.java:152-169 (segment walk), :558-599 (layout)
template <class F>
void ole_walk(const Group& g, int k, int rl, int ru, F&& f) {
  int boff = g.ptr[k], blen = g.ptr[k + 1] - g.ptr[k];
  int seg = 0;
  for (int bix = 0; bix < blen; bix += g.data[boff + bix] + 1, seg++) {
    int n = g.data[boff + bix];
    int base = seg * BITMAP_BLOCK_SZ;
    if (base >= ru) break;
    for (int j = 1; j <= n; j++) {
      int r = base + g.data[boff + bix + j];
      if (r >= rl && r < ru) f(r);
    }
  }
}

// visit (row, tupleId) of all non-default rows in [rl,ru)
template <class F>
void walk_rows(const Group& g, int rl, int ru, F&& f) {
  switch (g.type) {
    case G_DDC:
      for (int r = rl; r < ru; r++) f(r, g.map.get(r));
      break;
    case G_SDC: {
      if (g.off.type == OCL_OFF_EMPTY) break;
      OffIter it(g.off);
      // the reference iterates until value() == offsetToLast (e.g. CG/ColGroupSDCZeros.java:222-315)
      while (true) {
        if (it.row >= ru) break;
        if (it.row >= rl) f(it.row, g.single ? 0 : g.map.get(it.dataIndex));
        if (it.atLast()) break;
        it.next();
      }
      break;
    }
    case G_RLE:
      for (int k = 0; k < g.nVals; k++)
        rle_walk(g, k, rl, ru, [&](int a, int b) { for (int r = a; r < b; r++) f(r, k); });
      break;
    case G_OLE:
      for (int k = 0; k < g.nVals; k++) ole_walk(g, k, rl, ru, [&](int r) { f(r, k); });
      break;
    default: break;
  }
}

// AColGroupValue.getCounts: DDC/SDC histogram of the map (CG/mapping/MapToByte.java:168-188),
// RLE CG/ColGroupRLE.java:259-265, OLE CG/ColGroupOLE.java:152-169, SDCSingle {#offsets}
void group_counts(const ocl_matrix* m, const Group& g, std::vector<int64_t>& counts) {
  counts.assign(std::max(g.nVals, 1), 0);
  switch (g.type) {
    case G_DDC:
      for (int64_t r = 0; r < g.map.size; r++) counts[g.map.get(r)]++;
      break;
    case G_SDC:
      if (g.single) {
        int64_t n = 0;
        walk_rows(g, 0, m->nRows, [&](int, int) { n++; });
        counts[0] = n;
      } else
        for (int64_t r = 0; r < g.map.size; r++) counts[g.map.get(r)]++;
      break;
    case G_RLE:
      for (int k = 0; k < g.nVals; k++)
        for (int p = g.ptr[k]; p < g.ptr[k + 1]; p += 2) counts[k] += g.data[p + 1];
      break;
    case G_OLE:
      for (int k = 0; k < g.nVals; k++) {
        int boff = g.ptr[k], blen = g.ptr[k + 1] - g.ptr[k];
        for (int bix = 0; bix < blen; bix += g.data[boff + bix] + 1) counts[k] += g.data[boff + bix];
      }
      break;
    default: break;
  }
}

/* ---------------------------------------------------------------------------------------------
 * constV filtering -- C/lib/CLALibUtils.java:188-206 (filterGroups), CG/ColGroupSDC.java:483-489
 * (extractCommon: default tuple goes to constV, dictionary has the default subtracted),
 * CG/ColGroupConst.java:330-352 (addToCommon).
 * A "view" is a group with possibly replaced dictionary.
 * ------------------------------------------------------------------------------------------- */
struct View {
  const Group* g;
  std::vector<double> dict;  // effective dictionary
};

bool should_prefilter(const ocl_matrix* m) {  // C/lib/CLALibUtils.java:90-98
  for (auto& g : m->groups)
    if (g.type == G_CONST || g.type == G_EMPTY || (g.type == G_SDC && !g.def.empty())) return true;
  return false;
}

void filter_groups(const ocl_matrix* m, std::vector<View>& out, std::vector<double>& constV) {
  constV.assign(m->nCols, 0.0);
  for (auto& g : m->groups) {
    if (g.type == G_EMPTY) continue;
    if (g.type == G_CONST) {
      for (int j = 0; j < g.gCols(); j++) constV[g.cols[j]] += g.dict[j];
      continue;
    }
    View v{&g, g.dict};
    if (g.type == G_SDC && !g.def.empty()) {
      int gc = g.gCols();
      for (int j = 0; j < gc; j++) constV[g.cols[j]] += g.def[j];
      for (int k = 0; k < g.nVals; k++)
        for (int j = 0; j < gc; j++) v.dict[(size_t)k * gc + j] -= g.def[j];  // subtractTuple
    }
    out.push_back(std::move(v));
  }
}

/* ---------------------------------------------------------------------------------------------
 * decompress-and-sum of "RMM result groups": each view carries a table P [nVals x pc] and writes to
 * output columns outCols[0..pc). C/lib/CLALibDecompress.java:310-357,401-444: row blocks of
 * max(nRows/k,512), inner blocks of max(32768/ncol,128) rows, groups in list order, constV last.
 * ------------------------------------------------------------------------------------------- */
struct OutGroup {
  const Group* g;
  const double* P;     // [nVals x pc] (UNC: [nRows x pc])
  int pc;
  const int* outCols;  // nullptr => 0..pc-1
};

void decompress_block(const std::vector<OutGroup>& ogs, const double* constRow, double* out, int outCols,
                      int rl, int ru) {
  for (auto& og : ogs) {
    const Group& g = *og.g;
    const int pc = og.pc;
    if (g.type == G_UNC) {  // CG/ColGroupUncompressed.java:313-390
      for (int r = rl; r < ru; r++) {
        double* c = out + (size_t)r * outCols;
        const double* p = og.P + (size_t)r * pc;
        if (og.outCols) for (int j = 0; j < pc; j++) c[og.outCols[j]] += p[j];
        else for (int j = 0; j < pc; j++) c[j] += p[j];
      }
      continue;
    }
    // DDC CG/ColGroupDDC.java:137-225; SDCZeros CG/ColGroupSDCZeros.java:122-315; RLE CG/ColGroupRLE.java:104-141
    walk_rows(g, rl, ru, [&](int r, int k) {
      double* c = out + (size_t)r * outCols;
      const double* p = og.P + (size_t)k * pc;
      if (og.outCols) for (int j = 0; j < pc; j++) c[og.outCols[j]] += p[j];
      else for (int j = 0; j < pc; j++) c[j] += p[j];
    });
  }
  if (constRow)  // CLALibDecompress.java:427-434
    for (int r = rl; r < ru; r++) {
      double* c = out + (size_t)r * outCols;
      for (int j = 0; j < outCols; j++) c[j] += constRow[j];
    }
}

void decompress_dense(const std::vector<OutGroup>& ogs, const double* constRow, double* out, int nRows,
                      int outCols, int k) {
  const int blklen = std::max(nRows / std::max(k, 1), 512);
  const int inner = std::max(32768 / std::max(outCols, 1), 128);
  const int nblk = (nRows + blklen - 1) / blklen;
#pragma omp parallel for schedule(dynamic, 1) num_threads(std::max(k, 1))
  for (int b = 0; b < nblk; b++) {
    int rl = b * blklen, ru = std::min(nRows, rl + blklen);
    for (int r0 = rl; r0 < ru; r0 += inner) decompress_block(ogs, constRow, out, outCols, r0, std::min(ru, r0 + inner));
  }
}

// CG/dictionary/Dictionary.java:893-908 preaggValuesFromDense: ret[k, i] += dict[k,h] * V[cols[h], i]
void preagg_values_from_dense(const std::vector<double>& dict, int nVals, const std::vector<int>& cols,
                              const double* V, int vCols, std::vector<double>& ret) {
  const int cz = (int)cols.size();
  ret.assign((size_t)nVals * vCols, 0.0);
  for (int k = 0; k < nVals; k++)
    for (int h = 0; h < cz; h++) {
      const double v = dict[(size_t)k * cz + h];
      if (v != 0) {
        const double* b = V + (size_t)cols[h] * vCols;
        double* r = &ret[(size_t)k * vCols];
        for (int i = 0; i < vCols; i++) r[i] += v * b[i];
      }
    }
}

/* C/lib/CLALibRightMultBy.java:208-258 (RMM) */
void rmm(const ocl_matrix* m, const double* V, int vCols, double* out, int k) {
  const int nRows = m->nRows;
  std::memset(out, 0, sizeof(double) * (size_t)nRows * vCols);
  std::vector<View> views;
  std::vector<double> constV;
  filter_groups(m, views, constV);
  const bool filtered = should_prefilter(m);
  std::vector<std::vector<double>> P(views.size());
  // RMMParallel: one task per group (C/lib/CLALibRightMultBy.java:273-294)
#pragma omp parallel for schedule(dynamic, 1) num_threads(std::max(k, 1))
  for (size_t gi = 0; gi < views.size(); gi++) {
    const Group& g = *views[gi].g;
    if (g.type == G_UNC) {  // CG/ColGroupUncompressed.java:888-927: dense [nRows x gCols] x V[cols,:]
      const int gc = g.gCols();
      P[gi].assign((size_t)nRows * vCols, 0.0);
      for (int r = 0; r < nRows; r++)
        for (int h = 0; h < gc; h++) {
          const double v = g.dense[(size_t)r * gc + h];
          const double* b = V + (size_t)g.cols[h] * vCols;
          double* o = &P[gi][(size_t)r * vCols];
          for (int i = 0; i < vCols; i++) o[i] += v * b[i];
        }
    } else
      preagg_values_from_dense(views[gi].dict, g.nVals, g.cols, V, vCols, P[gi]);  // CG/ADictBasedColGroup.java:246-275
  }
  std::vector<double> constRow;
  if (filtered) {  // constV x V, CLALibRightMultBy.java:247-252
    constRow.assign(vCols, 0.0);
    bool any = false;
    for (int c = 0; c < m->nCols; c++)
      if (constV[c] != 0)
        for (int i = 0; i < vCols; i++) constRow[i] += constV[c] * V[(size_t)c * vCols + i];
    for (double x : constRow) any |= (x != 0);
    if (!any) constRow.clear();
  }
  std::vector<OutGroup> ogs;
  for (size_t gi = 0; gi < views.size(); gi++) ogs.push_back({views[gi].g, P[gi].data(), vCols, nullptr});
  decompress_dense(ogs, constRow.empty() ? nullptr : constRow.data(), out, nRows, vCols, k);
}

/* plain decompress: C/lib/CLALibDecompress.java:56-251 on the filtered groups + constV */
void decompress(const ocl_matrix* m, double* out, int k) {
  std::memset(out, 0, sizeof(double) * (size_t)m->nRows * m->nCols);
  std::vector<View> views;
  std::vector<double> constV;
  filter_groups(m, views, constV);
  std::vector<OutGroup> ogs;
  for (auto& v : views)
    ogs.push_back({v.g, v.g->type == G_UNC ? v.g->dense.data() : v.dict.data(), v.g->gCols(), v.g->cols.data()});
  bool any = false;
  for (double x : constV) any |= (x != 0);
  decompress_dense(ogs, any ? constV.data() : nullptr, out, m->nRows, m->nCols, k);
}

/* ---------------------------------------------------------------------------------------------
 * LMM -- C/lib/CLALibLeftMultBy.java:286-346 (LMM), :367-405 (NoTempOut split), :731-790
 * (LMMWithPreAggDense), CG/APreAgg.java:312-322 (mmWithDictionary), CG/ColGroupUtils.java:283-311.
 * left = Yt [q x nRows] row-major.
 * ------------------------------------------------------------------------------------------- */

// APreAgg.preAggregateDense: preAgg[(i-rl)*nVals + id] += left[i, r] for r in [cl,cu)
// DDC: CG/mapping/AMapToData.java:214-330; SDC: CG/offset/AOffset.java:288-420; RLE: CG/ColGroupRLE.java:759-796
void preaggregate_dense(const Group& g, const double* left, int nRows, double* preAgg, int rl, int ru, int cl,
                        int cu) {
  const int nv = g.nVals;
  walk_rows(g, cl, cu, [&](int r, int id) {
    for (int i = rl; i < ru; i++) preAgg[(size_t)(i - rl) * nv + id] += left[(size_t)i * nRows + r];
  });
}

void lmm_with_preagg(const std::vector<View>& pa, const double* left, int nRows, double* out, int nColsOut, int rl,
                     int ru, int cl, int cu, int off, int skip, double* rowSum) {
  const int colBZ = 2048, rowBlockSize = 4, colGroupBlocking = 4;
  const int nG = (int)pa.size();
  std::vector<std::vector<double>> preAgg(colGroupBlocking);
  std::vector<double> tmp;
  for (int rlt = rl; rlt < ru; rlt += rowBlockSize) {
    const int rut = std::min(rlt + rowBlockSize, ru);
    for (int gl = off; gl < nG; gl += colGroupBlocking * skip) {
      const int gu = std::min(gl + colGroupBlocking * skip, nG);
      for (int j = gl, p = 0; j < gu; j += skip, p++) preAgg[p].assign((size_t)(rut - rlt) * pa[j].g->nVals, 0.0);
      for (int clt = cl; clt < cu; clt += colBZ) {
        const int cut = std::min(clt + colBZ, cu);
        for (int j = gl, p = 0; j < gu; j += skip, p++)
          preaggregate_dense(*pa[j].g, left, nRows, preAgg[p].data(), rlt, rut, clt, cut);
        if (gu == nG && rowSum)  // :773-774
          for (int i = rlt; i < rut; i++)
            for (int c = clt; c < cut; c++) rowSum[i] += left[(size_t)i * nRows + c];
      }
      for (int j = gl, p = 0; j < gu; j += skip, p++) {  // postMultiply
        const Group& g = *pa[j].g;
        const int gc = g.gCols(), nv = g.nVals;
        tmp.assign((size_t)(rut - rlt) * gc, 0.0);
        for (int i = 0; i < rut - rlt; i++)
          for (int kk = 0; kk < nv; kk++) {
            const double a = preAgg[p][(size_t)i * nv + kk];
            if (a != 0)
              for (int c = 0; c < gc; c++) tmp[(size_t)i * gc + c] += a * pa[j].dict[(size_t)kk * gc + c];
          }
        for (int i = 0; i < rut - rlt; i++)
          for (int c = 0; c < gc; c++) out[(size_t)(rlt + i) * nColsOut + g.cols[c]] += tmp[(size_t)i * gc + c];
      }
    }
  }
}

void lmm(const ocl_matrix* m, const double* left, int q, double* out, int k) {
  const int nRows = m->nRows, nCols = m->nCols;
  std::memset(out, 0, sizeof(double) * (size_t)q * nCols);
  std::vector<View> views;
  std::vector<double> constV;
  filter_groups(m, views, constV);
  const bool filtered = should_prefilter(m);
  std::vector<View> pa, npa;
  for (auto& v : views) (v.g->type == G_UNC ? npa : pa).push_back(v);
  std::vector<double> rowSums(q, 0.0);
  k = std::max(k, 1);
  const int s = std::max(1, std::min((int)pa.size(), k));
  const int rowBlockSize = std::max(q / k, 1);
  // pre-agg groups: strided subsets, one task each (writes to disjoint output columns unless overlapping)
  // the reference writes directly into ret when groups do not overlap; disjoint columns make this race free.
  // overlapping groups share output columns: private results per task, summed afterwards
  // (LMMParallelTempOut, CLALibLeftMultBy.java:442-493)
  std::vector<int> cover(nCols, 0);
  bool overlapping = false;
  for (auto& v : pa)
    for (int c : v.g->cols) overlapping |= (++cover[c] > 1);
  std::vector<std::vector<double>> tmpOut(overlapping ? s : 0);
#pragma omp parallel for schedule(dynamic, 1) num_threads(k)
  for (int off = 0; off < s; off++) {
    double* dst = out;
    if (overlapping) {
      tmpOut[off].assign((size_t)q * nCols, 0.0);
      dst = tmpOut[off].data();
    }
    for (int blo = 0; blo < q; blo += rowBlockSize)
      lmm_with_preagg(pa, left, nRows, dst, nCols, blo, std::min(blo + rowBlockSize, q), 0, nRows, off, s, nullptr);
  }
  for (auto& t : tmpOut)
    for (size_t i = 0; i < (size_t)q * nCols; i++) out[i] += t[i];
  if (filtered)  // separate rowSum task in the parallel variants (CLALibLeftMultBy.java:399-400)
    for (int i = 0; i < q; i++)
      for (int r = 0; r < nRows; r++) rowSums[i] += left[(size_t)i * nRows + r];
  // non-pre-agg (uncompressed) groups: CG/ColGroupUncompressed.java:429-539, column blocks of
  // max(ct/max(k,2), 64000) summed through temporaries (CLALibLeftMultBy.java:407-440)
  for (auto& v : npa) {
    const Group& g = *v.g;
    const int gc = g.gCols();
    const int cbs = std::max(nRows / std::max(k, 2), 64000);
    const int nb = (nRows + cbs - 1) / cbs;
    std::vector<std::vector<double>> tmps(nb);
#pragma omp parallel for schedule(dynamic, 1) num_threads(k)
    for (int b = 0; b < nb; b++) {
      tmps[b].assign((size_t)q * gc, 0.0);
      const int c0 = b * cbs, c1 = std::min(nRows, c0 + cbs);
      for (int i = 0; i < q; i++)
        for (int r = c0; r < c1; r++) {
          const double a = left[(size_t)i * nRows + r];
          if (a != 0)
            for (int c = 0; c < gc; c++) tmps[b][(size_t)i * gc + c] += a * g.dense[(size_t)r * gc + c];
        }
    }
    for (int b = 0; b < nb; b++)
      for (int i = 0; i < q; i++)
        for (int c = 0; c < gc; c++) out[(size_t)i * nCols + g.cols[c]] += tmps[b][(size_t)i * gc + c];
  }
  if (filtered)  // outerProduct(rowSums, constV): CLALibLeftMultBy.java:530-629
    for (int i = 0; i < q; i++)
      for (int c = 0; c < nCols; c++) out[(size_t)i * nCols + c] += rowSums[i] * constV[c];
}

/* ---------------------------------------------------------------------------------------------
 * TSMM -- C/lib/CLALibTSMM.java:59-166
 * ------------------------------------------------------------------------------------------- */

// DictLibMatrixMult.addToUpperTriangle: CG/dictionary/DictLibMatrixMult.java:47-54
inline void add_upper(int nCols, int row, int col, double* res, double val) {
  if (row == col) res[(size_t)row * nCols + col] += val + val;
  else if (row > col) res[(size_t)col * nCols + row] += val;
  else res[(size_t)row * nCols + col] += val;
}

// AColGroupCompressed.tsmmDense: CG/AColGroupCompressed.java:226-241
void tsmm_self(const View& v, const std::vector<int64_t>& counts, double* res, int nCols) {
  const Group& g = *v.g;
  const int gc = g.gCols();
  for (int k = 0; k < g.nVals; k++) {
    const double scale = (double)counts[k];
    for (int i = 0; i < gc; i++) {
      const double x = v.dict[(size_t)k * gc + i] * scale;
      if (x != 0)
        for (int j = i; j < gc; j++) res[(size_t)g.cols[i] * nCols + g.cols[j]] += x * v.dict[(size_t)k * gc + j];
    }
  }
}

// preAggregateThatIndexStructure (CG/APreAgg.java:87-117): table B[k_this, :] = sum over rows r with
// this.id(r) = k_this of that.dict[that.id(r), :]. Joint scans: CG/mapping/AMapToData.java:429-794,
// CG/ColGroupSDCZeros.java:682-753, CG/ColGroupRLE.java:835-956.  Realised through per-row ids.
void preagg_that(const ocl_matrix* m, const View& self, const View& that, std::vector<double>& B) {
  const int n = m->nRows, tc = that.g->gCols();
  std::vector<int32_t> idThis(n, -1);
  walk_rows(*self.g, 0, n, [&](int r, int k) { idThis[r] = k; });
  B.assign((size_t)self.g->nVals * tc, 0.0);
  walk_rows(*that.g, 0, n, [&](int r, int kt) {
    const int k = idThis[r];
    if (k >= 0)
      for (int j = 0; j < tc; j++) B[(size_t)k * tc + j] += that.dict[(size_t)kt * tc + j];
  });
}

// TSMMToUpperTriangle (DictLibMatrixMult.java:151-237,527-601): res += left^T * right into the upper triangle
void mm_to_upper(const double* left, const double* right, int commonDim, const std::vector<int>& rowsLeft,
                 const std::vector<int>& colsRight, double* res, int nCols) {
  const int ls = (int)rowsLeft.size(), rs = (int)colsRight.size();
  for (int k = 0; k < commonDim; k++)
    for (int i = 0; i < ls; i++) {
      const double vl = left[(size_t)k * ls + i];
      if (vl != 0)
        for (int j = 0; j < rs; j++) add_upper(nCols, rowsLeft[i], colsRight[j], res, vl * right[(size_t)k * rs + j]);
    }
}

// APreAgg.tsmmAPreAgg (CG/APreAgg.java:153-180): "this" = right group (h), lg = left group (g)
void tsmm_pair(const ocl_matrix* m, const View& lg, const View& rg, double* res, int nCols) {
  // shouldPreAggregateLeft (APreAgg.java:302-310): costRight = nvR*rCol < costLeft = nvL*lCol
  const double costR = (double)rg.g->nVals * rg.g->gCols(), costL = (double)lg.g->nVals * lg.g->gCols();
  std::vector<double> B;
  if (costR < costL) {  // this(=rg).preAggregateThatIndexStructure(lg): B[k_r, lcols]
    preagg_that(m, rg, lg, B);
    mm_to_upper(B.data(), rg.dict.data(), rg.g->nVals, lg.g->cols, rg.g->cols, res, nCols);
  } else {  // lg.preAggregateThatIndexStructure(this): B[k_l, rcols]
    preagg_that(m, lg, rg, B);
    mm_to_upper(lg.dict.data(), B.data(), lg.g->nVals, lg.g->cols, rg.g->cols, res, nCols);
  }
}

// LibMatrixMult.matrixMultTransposeSelf (dense, upper triangle by dot products) on the decompressed matrix
void dense_tsmm_upper(const double* X, int64_t n, int mcols, double* res, int k) {
#pragma omp parallel for schedule(dynamic, 1) num_threads(std::max(k, 1))
  for (int i = 0; i < mcols; i++)
    for (int j = i; j < mcols; j++) {
      double s = 0;
      for (int64_t r = 0; r < n; r++) s += X[r * mcols + i] * X[r * mcols + j];
      res[(size_t)i * mcols + j] = s;
    }
}

void tsmm(const ocl_matrix* m, double* out, int k, int allowFallback) {
  const int nCols = m->nCols, nRows = m->nRows;
  std::memset(out, 0, sizeof(double) * (size_t)nCols * nCols);
  bool hasUnc = false;
  for (auto& g : m->groups) hasUnc |= (g.type == G_UNC);
  if (hasUnc || (allowFallback && (int)m->groups.size() >= nCols)) {  // CLALibTSMM.java:73-77
    std::vector<double> X((size_t)nRows * nCols);
    decompress(m, X.data(), k);
    dense_tsmm_upper(X.data(), nRows, nCols, out, k);
  } else {
    std::vector<View> views;
    std::vector<double> constV;
    filter_groups(m, views, constV);
    const bool filtered = should_prefilter(m);
    const int nG = (int)views.size();
    std::vector<std::vector<int64_t>> counts(nG);
    for (int i = 0; i < nG; i++) group_counts(m, *views[i].g, counts[i]);
    // one task per group and per unordered pair (CLALibTSMM.java:135-154); private results summed
    std::vector<std::pair<int, int>> tasks;
    for (int i = 0; i < nG; i++) {
      tasks.push_back({i, i});
      for (int j = i + 1; j < nG; j++) tasks.push_back({i, j});
    }
    const int nt = std::max(k, 1);
    std::vector<std::vector<double>> priv(nt, std::vector<double>((size_t)nCols * nCols, 0.0));
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt)
    for (size_t t = 0; t < tasks.size(); t++) {
#ifdef _OPENMP
      double* res = priv[omp_get_thread_num()].data();
#else
      double* res = priv[0].data();
#endif
      if (tasks[t].first == tasks[t].second) tsmm_self(views[tasks[t].first], counts[tasks[t].first], res, nCols);
      else tsmm_pair(m, views[tasks[t].first], views[tasks[t].second], res, nCols);
    }
    for (int t = 0; t < nt; t++)
      for (size_t i = 0; i < (size_t)nCols * nCols; i++) out[i] += priv[t][i];
    if (filtered) {  // addCorrectionLayer: CLALibTSMM.java:156-166 with colSums of the filtered groups
      std::vector<double> cs(nCols, 0.0);
      for (int i = 0; i < nG; i++) {
        const Group& g = *views[i].g;
        for (int kk = 0; kk < g.nVals; kk++)
          for (int j = 0; j < g.gCols(); j++) cs[g.cols[j]] += views[i].dict[(size_t)kk * g.gCols() + j] * (double)counts[i][kk];
      }
      for (int row = 0; row < nCols; row++) {
        const double v1 = constV[row], v2 = cs[row] + constV[row] * nRows;
        for (int col = row; col < nCols; col++) out[(size_t)row * nCols + col] += v1 * cs[col] + v2 * constV[col];
      }
    }
  }
  // LibMatrixMult.copyUpperToLowerTriangle: runtime/matrix/data/LibMatrixMult.java:4769-4799
  for (int i = 0; i < nCols; i++)
    for (int j = i + 1; j < nCols; j++) out[(size_t)j * nCols + i] = out[(size_t)i * nCols + j];
}

/* mmchain -- C/lib/CLALibMMChain.java:92-146: RMM (dense u), optional w, transposed LMM */
void mmchain(const ocl_matrix* m, const double* v, const double* w, int ctype, double* out, int k) {
  if (ctype == OCL_CHAIN_XtXv && (int)m->groups.size() < 5 && m->nCols > 30) {  // :99-102
    std::vector<double> t((size_t)m->nCols * m->nCols);
    tsmm(m, t.data(), k, 1);
    for (int i = 0; i < m->nCols; i++) {
      double s = 0;
      for (int j = 0; j < m->nCols; j++) s += t[(size_t)i * m->nCols + j] * v[j];
      out[i] = s;
    }
    return;
  }
  std::vector<double> u(m->nRows);
  rmm(m, v, 1, u.data(), k);
  if (ctype == OCL_CHAIN_XtwXv)
    for (int r = 0; r < m->nRows; r++) u[r] *= w[r];
  lmm(m, u.data(), 1, out, k);
}

/* t(left) %*% right on two compressed blocks -- C/lib/CLALibLeftMultBy.java:100-112,170-284
 * (leftMultByCompressedTransposedMatrix): both sides are filtered to zero-default groups + constV; every pair
 * (left group lg, right group rg) adds t(lg) rg through rg.leftMultByAColGroup(lg) (CG/APreAgg.java:57-68,
 * 211-232): the side with the cheaper dictionary is pre-aggregated by the other side's index structure
 * (shouldPreAggregateLeft :302-310), then one small dictionary product; uncompressed groups on either side
 * (CG/APreAgg.java:234-248, CG/ColGroupUncompressed.java:732-827) go through their dense rows. Then the rank-1
 * corrections cL (x) colSums(right'), colSums(left') (x) cR and nRows * cL (x) cR (:206-214). */
struct RowSrc {  // a filtered group seen as "row r holds tuple id(r) of table T" (id -1: zero row)
  const double* T;
  int gc;
  std::vector<int32_t> id;
};
void row_src(const View& v, int n, RowSrc& rs) {
  const Group& g = *v.g;
  rs.gc = g.gCols();
  rs.id.assign(n, -1);
  if (g.type == G_UNC) {
    rs.T = g.dense.data();
    for (int r = 0; r < n; r++) rs.id[r] = r;
  } else {
    rs.T = v.dict.data();
    walk_rows(g, 0, n, [&](int r, int k) { rs.id[r] = k; });
  }
}

void tmm_pair(int n, const View& lg, const View& rg, double* res, int nColsOut) {
  const Group &L = *lg.g, &R = *rg.g;
  const int lc = L.gCols(), rc = R.gCols();
  if (L.type == G_UNC || R.type == G_UNC) {  // dense rows on one side: pre-aggregate them by the other side's ids
    RowSrc a, b;
    row_src(lg, n, a);
    row_src(rg, n, b);
    if (L.type == G_UNC && R.type != G_UNC) {  // APreAgg.leftMultByUncompressedColGroup: preAgg[lc x nVals_r] . D_r
      std::vector<double> pa((size_t)lc * R.nVals, 0.0);
      for (int r = 0; r < n; r++)
        if (b.id[r] >= 0)
          for (int i = 0; i < lc; i++) pa[(size_t)i * R.nVals + b.id[r]] += a.T[(size_t)r * lc + i];
      for (int i = 0; i < lc; i++)
        for (int k = 0; k < R.nVals; k++) {
          const double x = pa[(size_t)i * R.nVals + k];
          if (x != 0)
            for (int j = 0; j < rc; j++) res[(size_t)L.cols[i] * nColsOut + R.cols[j]] += x * rg.dict[(size_t)k * rc + j];
        }
    } else {  // right side dense: out[lcols, rcols] += sum_r tuple_l(r)^T row_r(r), row by row
      for (int r = 0; r < n; r++)
        if (a.id[r] >= 0 && b.id[r] >= 0)
          for (int i = 0; i < lc; i++) {
            const double x = a.T[(size_t)a.id[r] * lc + i];
            if (x != 0)
              for (int j = 0; j < rc; j++) res[(size_t)L.cols[i] * nColsOut + R.cols[j]] += x * b.T[(size_t)b.id[r] * rc + j];
          }
    }
    return;
  }
  ocl_matrix shape;  // preagg_that only reads the row count
  shape.nRows = n;
  shape.nCols = 0;
  std::vector<double> B;
  const double costR = (double)R.nVals * rc, costL = (double)L.nVals * lc;
  if (costR < costL) {  // left pre-aggregation: B[k_l, rcols] = sum of right tuples over rows with left id k_l
    preagg_that(&shape, lg, rg, B);
    for (int k = 0; k < L.nVals; k++)
      for (int i = 0; i < lc; i++) {
        const double x = lg.dict[(size_t)k * lc + i];
        if (x != 0)
          for (int j = 0; j < rc; j++) res[(size_t)L.cols[i] * nColsOut + R.cols[j]] += x * B[(size_t)k * rc + j];
      }
  } else {  // right pre-aggregation: B[k_r, lcols]
    preagg_that(&shape, rg, lg, B);
    for (int k = 0; k < R.nVals; k++)
      for (int i = 0; i < lc; i++) {
        const double x = B[(size_t)k * lc + i];
        if (x != 0)
          for (int j = 0; j < rc; j++) res[(size_t)L.cols[i] * nColsOut + R.cols[j]] += x * rg.dict[(size_t)k * rc + j];
      }
  }
}

// CLALibUtils.getColSum (C/lib/CLALibUtils.java:267-269) of filtered groups
void col_sums_filtered(const ocl_matrix* m, const std::vector<View>& views, std::vector<double>& cs) {
  cs.assign(m->nCols, 0.0);
  for (auto& v : views) {
    const Group& g = *v.g;
    const int gc = g.gCols();
    if (g.type == G_UNC) {
      for (int r = 0; r < m->nRows; r++)
        for (int j = 0; j < gc; j++) cs[g.cols[j]] += g.dense[(size_t)r * gc + j];
      continue;
    }
    std::vector<int64_t> counts;
    group_counts(m, g, counts);
    for (int k = 0; k < g.nVals; k++)
      for (int j = 0; j < gc; j++) cs[g.cols[j]] += v.dict[(size_t)k * gc + j] * (double)counts[k];
  }
}

void tmm(const ocl_matrix* left, const ocl_matrix* right, double* out, int k) {
  const int rl = left->nCols, cr = right->nCols, sd = right->nRows;
  std::memset(out, 0, sizeof(double) * (size_t)rl * cr);
  std::vector<View> fL, fR;
  std::vector<double> cL, cR;
  filter_groups(left, fL, cL);
  filter_groups(right, fR, cR);
  const bool containsLeft = should_prefilter(left), containsRight = should_prefilter(right);
  const int nt = std::max(k, 1);
  // one task per left group with a private result, summed afterwards (:186-200, :216-230)
  std::vector<std::vector<double>> priv(nt, std::vector<double>((size_t)rl * cr, 0.0));
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt)
  for (size_t j = 0; j < fL.size(); j++) {
#ifdef _OPENMP
    double* res = priv[omp_get_thread_num()].data();
#else
    double* res = priv[0].data();
#endif
    for (size_t i = 0; i < fR.size(); i++) tmm_pair(sd, fL[j], fR[i], res, cr);
  }
  if (containsLeft && containsRight)  // outerProductWithScaling
    for (int i = 0; i < rl; i++)
      for (int j = 0; j < cr; j++) out[(size_t)i * cr + j] += cL[i] * cR[j] * sd;
  if (containsLeft) {
    std::vector<double> cs;
    col_sums_filtered(right, fR, cs);
    for (int i = 0; i < rl; i++)
      for (int j = 0; j < cr; j++) out[(size_t)i * cr + j] += cL[i] * cs[j];
  }
  if (containsRight) {
    std::vector<double> cs;
    col_sums_filtered(left, fL, cs);
    for (int i = 0; i < rl; i++)
      for (int j = 0; j < cr; j++) out[(size_t)i * cr + j] += cs[i] * cR[j];
  }
  for (int t = 0; t < nt; t++)
    for (size_t i = 0; i < (size_t)rl * cr; i++) out[i] += priv[t][i];
}

template <class T>
std::vector<T> vec(const T* p, size_t n) {
  return p ? std::vector<T>(p, p + n) : std::vector<T>();
}

void fill_map(Map& mp, int type, const void* a, const void* b, int64_t size) {
  mp.type = type;
  mp.size = size;
  switch (type) {
    case OCL_MAP_BIT: mp.bits = vec((const uint64_t*)a, (size_t)((size + 63) / 64)); break;
    case OCL_MAP_UBYTE:
    case OCL_MAP_BYTE: mp.b = vec((const uint8_t*)a, (size_t)size); break;
    case OCL_MAP_CHAR: mp.c = vec((const uint16_t*)a, (size_t)size); break;
    case OCL_MAP_CHAR_BYTE:
      mp.c = vec((const uint16_t*)a, (size_t)size);
      mp.b = vec((const uint8_t*)b, (size_t)size);
      break;
    case OCL_MAP_INT: mp.i = vec((const int32_t*)a, (size_t)size); break;
    default: break;
  }
}

Group base_group(GType t, const int32_t* cols, int gCols, const double* dict, int nVals) {
  Group g;
  g.type = t;
  g.cols.assign(cols, cols + gCols);
  g.nVals = nVals;
  if (dict) g.dict.assign(dict, dict + (size_t)nVals * gCols);
  return g;
}

}  // namespace

extern "C" {

// CG/mapping/MapToFactory.java:102-117
int ocl_map_type_for(int64_t size, int64_t unique) {
  if (unique <= 1) return OCL_MAP_ZERO;
  if (unique == 2 && size > 32) return OCL_MAP_BIT;
  if (unique <= 128) return OCL_MAP_UBYTE;
  if (unique <= 256) return OCL_MAP_BYTE;
  if (unique <= 65536) return OCL_MAP_CHAR;
  if (unique <= 8388608) return OCL_MAP_CHAR_BYTE;
  return OCL_MAP_INT;
}

// CG/ColGroupOLE.java:558-599 genOffsetBitmap
int64_t ocl_ole_gen_offset_bitmap(const int32_t* offsets, int64_t len, uint16_t* out, int64_t cap) {
  if (!offsets || len == 0) return -1;
  const int lastOffset = offsets[len - 1];
  const int numBlocks = lastOffset / BITMAP_BLOCK_SZ + 1;
  std::vector<int> blockLengths(numBlocks, 0);
  for (int64_t ix = 0; ix < len; ix++) blockLengths[offsets[ix] / BITMAP_BLOCK_SZ]++;
  int64_t total = numBlocks;
  for (int b = 0; b < numBlocks; b++) total += blockLengths[b];
  int64_t inputIx = 0, blockStartIx = 0;
  for (int b = 0; b < numBlocks; b++) {
    const int sz = blockLengths[b];
    if (blockStartIx < cap) out[blockStartIx] = (uint16_t)sz;
    for (int i = 0; i < sz; i++)
      if (blockStartIx + i + 1 < cap) out[blockStartIx + i + 1] = (uint16_t)(offsets[inputIx + i] % BITMAP_BLOCK_SZ);
    inputIx += sz;
    blockStartIx += sz + 1;
  }
  return total;
}

// CG/ColGroupRLE.java:1073-1157 genRLEBitmap
int64_t ocl_rle_gen_bitmap(const int32_t* offsets, int64_t len, uint16_t* out, int64_t cap) {
  if (!offsets || len == 0) return -1;
  const int CM = 65535;
  std::vector<uint16_t> buf;
  int lastRunEnd = 0, curRunOff, curRunLen = 0;
  int firstOff = offsets[0];
  while (firstOff > CM) {
    buf.push_back((uint16_t)CM);
    buf.push_back(0);
    firstOff -= CM;
    lastRunEnd += CM;
  }
  curRunOff = firstOff;
  curRunLen = 1;
  for (int64_t i = 1; i < len; i++) {
    const int absOffset = offsets[i];
    const int curRunEnd = lastRunEnd + curRunOff + curRunLen;
    if (absOffset > curRunEnd || curRunLen >= CM) {
      buf.push_back((uint16_t)curRunOff);
      buf.push_back((uint16_t)curRunLen);
      lastRunEnd = curRunEnd;
      curRunOff = absOffset - lastRunEnd;
      while (curRunOff > CM) {
        buf.push_back((uint16_t)CM);
        buf.push_back(0);
        lastRunEnd += CM;
        curRunOff -= CM;
      }
      curRunLen = 1;
    } else
      curRunLen++;
  }
  buf.push_back((uint16_t)curRunOff);
  buf.push_back((uint16_t)curRunLen);
  for (size_t i = 0; i < buf.size() && (int64_t)i < cap; i++) out[i] = buf[i];
  return (int64_t)buf.size();
}

namespace {
// utils/MemoryEstimates.java:68-105
double byte_array_cost(int64_t length) {
  double size = 8 + 20;
  if (length <= 4) size += 4;
  else {
    size += length;
    double diff = (double)((length - 4) % 8);
    if (diff > 0) size += 8 - diff;
  }
  return size;
}
double char_array_cost(int64_t length) {
  double size = 8 + 20;
  if (length <= 2) size += 4;
  else {
    size += length * 2;
    double diff = (double)((length * 2 - 4) % 8);
    if (diff > 0) size += 8 - diff;
  }
  return size;
}
// CG/offset/OffsetByte.java:100-104, OffsetChar.java:88-92 (the double sum is truncated to long)
int64_t est_byte(int64_t n) { return (int64_t)(16 + 4 + 4 + 4 + 8 + byte_array_cost(n)); }
int64_t est_char(int64_t n) { return (int64_t)(16 + 4 + 4 + 8 + char_array_cost(n)); }
// OffsetFactory.java:228-234
int correction(int range, int size, int maxv1) { return std::max(range - size * maxv1, 0) / maxv1; }
int64_t calc_size(const int32_t* idx, int64_t n, int offMax) {  // OffsetFactory.java:285-294
  int64_t endSize = 0;
  int ov = idx[0];
  for (int64_t i = 1; i < n; i++) {
    endSize += 1 + (idx[i] - ov - 1) / offMax;
    ov = idx[i];
  }
  return endSize;
}
}  // namespace

// CG/offset/OffsetFactory.java:105-149 (createOffset), :238-283 (createByte), :296-338 (createChar)
int64_t ocl_offset_create(const int32_t* idx, int64_t n, int32_t* type, int32_t* first, int32_t* last, void* out,
                          int64_t cap, int32_t* flags) {
  *flags = 0;
  const int64_t endLength = n - 1;
  if (endLength < 0) { *type = OCL_OFF_EMPTY; *first = *last = 0; return 0; }
  *first = idx[0];
  *last = idx[n - 1];
  if (endLength == 0) { *type = OCL_OFF_SINGLE; return 0; }
  if (endLength == 1) { *type = OCL_OFF_TWO; return 0; }
  const int range = idx[n - 1] - idx[0];
  const int corrB = correction(range, (int)endLength, 256);
  const int corrC = correction(range, (int)endLength, 65535);
  const bool useByte = est_byte(endLength + corrB) < est_char(endLength + corrC);
  const int maxV = useByte ? BYTE_MAXV : CHAR_MAXV;
  const int64_t endSize = calc_size(idx, n, maxV);
  const bool noZero = endSize == n - 1;
  *type = useByte ? OCL_OFF_BYTE : OCL_OFF_CHAR;
  if (endSize > cap) return endSize;
  uint8_t* ob = (uint8_t*)out;
  uint16_t* oc = (uint16_t*)out;
  if (useByte) std::memset(ob, 0, (size_t)endSize);
  else std::memset(oc, 0, (size_t)endSize * 2);
  int ov = idx[0];
  int64_t p = 0;
  bool noOverHalf = true;
  for (int64_t i = 1; i < n; i++) {
    const int nv = idx[i], offsetSize = nv - ov;
    int store;
    if (noZero) store = offsetSize % (maxV + 1);
    else {
      const int div = offsetSize / maxV, mod = offsetSize % maxV;
      if (mod == 0) { p += div - 1; store = maxV; }
      else { p += div; store = mod; }
    }
    if (useByte) ob[p++] = (uint8_t)store;
    else oc[p++] = (uint16_t)store;
    ov = nv;
  }
  if (useByte)
    for (int64_t i = 0; i < endSize; i++) if ((int8_t)ob[i] < 1) noOverHalf = false;  // OffsetFactory.getNoOverHalf
  *flags = (noZero ? 1 : 0) | ((useByte && noOverHalf) ? 2 : 0);
  return endSize;
}

int64_t ocl_offset_decode(int32_t type, int32_t first, int32_t last, const void* data, int64_t len, int32_t* rows,
                          int64_t cap) {
  Offset o;
  o.type = type; o.first = first; o.last = last;
  if (type == OCL_OFF_BYTE) o.b = vec((const uint8_t*)data, (size_t)len);
  if (type == OCL_OFF_CHAR) o.c = vec((const uint16_t*)data, (size_t)len);
  if (type == OCL_OFF_EMPTY) return 0;
  OffIter it(o);
  int64_t n = 0;
  while (true) {
    if (n < cap) rows[n] = it.row;
    n++;
    if (it.atLast()) break;
    it.next();
  }
  return n;
}

void ocl_map_decode(int32_t type, const void* data, const void* data2, int64_t size, int32_t* ids) {
  Map mp;
  fill_map(mp, type, data, data2, size);
  for (int64_t r = 0; r < size; r++) ids[r] = mp.get(r);
}

ocl_matrix* ocl_create(int32_t nRows, int32_t nCols) {
  ocl_matrix* m = new ocl_matrix();
  m->nRows = nRows;
  m->nCols = nCols;
  return m;
}
void ocl_destroy(ocl_matrix* m) { delete m; }

int ocl_add_ddc(ocl_matrix* m, const int32_t* cols, int32_t gCols, const double* dict, int32_t nVals, int32_t mapType,
                const void* map, const void* map2, int64_t mapSize) {
  Group g = base_group(G_DDC, cols, gCols, dict, nVals);
  fill_map(g.map, mapType, map, map2, mapSize);
  m->groups.push_back(std::move(g));
  return (int)m->groups.size() - 1;
}

int ocl_add_sdc(ocl_matrix* m, const int32_t* cols, int32_t gCols, const double* dict, int32_t nVals,
                const double* defaultTuple, int32_t offType, int32_t first, int32_t last, const void* offData,
                int64_t offLen, int32_t mapType, const void* map, const void* map2, int64_t mapSize) {
  Group g = base_group(G_SDC, cols, gCols, dict, nVals);
  if (defaultTuple) g.def.assign(defaultTuple, defaultTuple + gCols);
  g.off.type = offType; g.off.first = first; g.off.last = last;
  if (offType == OCL_OFF_BYTE) g.off.b = vec((const uint8_t*)offData, (size_t)offLen);
  if (offType == OCL_OFF_CHAR) g.off.c = vec((const uint16_t*)offData, (size_t)offLen);
  g.single = (map == nullptr);
  if (!g.single) fill_map(g.map, mapType, map, map2, mapSize);
  m->groups.push_back(std::move(g));
  return (int)m->groups.size() - 1;
}

int ocl_add_rle(ocl_matrix* m, const int32_t* cols, int32_t gCols, const double* dict, int32_t nVals,
                const int32_t* ptr, const uint16_t* data, int64_t dataLen) {
  Group g = base_group(G_RLE, cols, gCols, dict, nVals);
  g.ptr.assign(ptr, ptr + nVals + 1);
  g.data = vec(data, (size_t)dataLen);
  m->groups.push_back(std::move(g));
  return (int)m->groups.size() - 1;
}

int ocl_add_ole(ocl_matrix* m, const int32_t* cols, int32_t gCols, const double* dict, int32_t nVals,
                const int32_t* ptr, const uint16_t* data, int64_t dataLen) {
  Group g = base_group(G_OLE, cols, gCols, dict, nVals);
  g.ptr.assign(ptr, ptr + nVals + 1);
  g.data = vec(data, (size_t)dataLen);
  m->groups.push_back(std::move(g));
  return (int)m->groups.size() - 1;
}

int ocl_add_uncompressed(ocl_matrix* m, const int32_t* cols, int32_t gCols, const double* values) {
  Group g = base_group(G_UNC, cols, gCols, nullptr, 0);
  g.dense.assign(values, values + (size_t)m->nRows * gCols);
  m->groups.push_back(std::move(g));
  return (int)m->groups.size() - 1;
}

int ocl_add_const(ocl_matrix* m, const int32_t* cols, int32_t gCols, const double* tuple) {
  Group g = base_group(G_CONST, cols, gCols, tuple, 1);
  m->groups.push_back(std::move(g));
  return (int)m->groups.size() - 1;
}

int ocl_add_empty(ocl_matrix* m, const int32_t* cols, int32_t gCols) {
  Group g = base_group(G_EMPTY, cols, gCols, nullptr, 0);
  m->groups.push_back(std::move(g));
  return (int)m->groups.size() - 1;
}

int32_t ocl_num_groups(const ocl_matrix* m) { return (int32_t)m->groups.size(); }

int64_t ocl_compressed_bytes(const ocl_matrix* m) {
  int64_t s = 0;
  for (auto& g : m->groups) {
    s += (int64_t)g.dict.size() * 8 + (int64_t)g.dense.size() * 8 + (int64_t)g.data.size() * 2 + (int64_t)g.ptr.size() * 4;
    s += (int64_t)g.map.bits.size() * 8 + (int64_t)g.map.b.size() + (int64_t)g.map.c.size() * 2 + (int64_t)g.map.i.size() * 4;
    s += (int64_t)g.off.b.size() + (int64_t)g.off.c.size() * 2;
  }
  return s;
}

void ocl_group_row_ids(const ocl_matrix* m, int32_t gi, int32_t* ids) {
  const Group& g = m->groups[gi];
  for (int r = 0; r < m->nRows; r++) ids[r] = (g.type == G_UNC) ? r : (g.type == G_CONST ? 0 : -1);
  walk_rows(g, 0, m->nRows, [&](int r, int k) { ids[r] = k; });
}

void ocl_group_counts(const ocl_matrix* m, int32_t gi, int64_t* counts) {
  std::vector<int64_t> c;
  group_counts(m, m->groups[gi], c);
  for (int k = 0; k < m->groups[gi].nVals; k++) counts[k] = c[k];
}

void ocl_decompress(const ocl_matrix* m, double* out, int k) { decompress(m, out, k); }
void ocl_rmm(const ocl_matrix* m, const double* V, int32_t vCols, double* out, int k) { rmm(m, V, vCols, out, k); }
void ocl_lmm(const ocl_matrix* m, const double* Yt, int32_t yRows, double* out, int k) { lmm(m, Yt, yRows, out, k); }
void ocl_tsmm(const ocl_matrix* m, double* out, int k, int allowFallback) { tsmm(m, out, k, allowFallback); }
void ocl_tmm(const ocl_matrix* left, const ocl_matrix* right, double* out, int k) { tmm(left, right, out, k); }
void ocl_mmchain(const ocl_matrix* m, const double* v, const double* w, int ctype, double* out, int k) {
  mmchain(m, v, w, ctype, out, k);
}

void ocl_dense_rmm_ld(const double* X, int64_t n, int32_t m, const double* V, int32_t vCols, double* out) {
#pragma omp parallel for
  for (int64_t r = 0; r < n; r++)
    for (int j = 0; j < vCols; j++) {
      long double s = 0;
      for (int c = 0; c < m; c++) s += (long double)X[r * m + c] * (long double)V[(size_t)c * vCols + j];
      out[r * vCols + j] = (double)s;
    }
}
void ocl_dense_lmm_ld(const double* X, int64_t n, int32_t m, const double* Yt, int32_t q, double* out) {
#pragma omp parallel for collapse(2)
  for (int i = 0; i < q; i++)
    for (int c = 0; c < m; c++) {
      long double s = 0;
      for (int64_t r = 0; r < n; r++) s += (long double)Yt[(size_t)i * n + r] * (long double)X[r * m + c];
      out[(size_t)i * m + c] = (double)s;
    }
}
void ocl_dense_tsmm_ld(const double* X, int64_t n, int32_t m, double* out) {
#pragma omp parallel for collapse(2)
  for (int i = 0; i < m; i++)
    for (int j = 0; j < m; j++) {
      if (j < i) continue;
      long double s = 0;
      for (int64_t r = 0; r < n; r++) s += (long double)X[r * m + i] * (long double)X[r * m + j];
      out[(size_t)i * m + j] = out[(size_t)j * m + i] = (double)s;
    }
}

int ocl_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"
