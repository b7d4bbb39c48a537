// systemds_cla.hpp -- C++ host-side mirror of the reference's operator API for the compressed matrix products,
// on top of the C ABI in systemds_cla.h. Header only.
//
// The reference's host language is Java; where no JVM is available this header is the compiled-language host
// layer: the same class and method names, argument meaning and error behaviour as
//   runtime/compress/CompressedMatrixBlock.java, runtime/compress/colgroup/ColGroup*.java,
//   colgroup/mapping/MapToFactory.java, colgroup/offset/OffsetFactory.java and
//   runtime/compress/lib/CLALib{RightMultBy,LeftMultBy,TSMM,MMChain,Decompress}.java
// (paths below src/main/java/org/apache/sysds/). Failures surface as DMLCompressionException, as in the reference.
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>
#include "systemds_cla.h"

namespace sysds {
namespace cla {

struct DMLCompressionException : std::runtime_error {
  int64_t code;
  DMLCompressionException(int64_t c, const std::string& what) : std::runtime_error(what), code(c) {}
};

inline int64_t check(int64_t rc, const char* where) {
  if (rc < 0) {
    char buf[1024];
    cla_last_error(buf, sizeof(buf));
    throw DMLCompressionException(rc, std::string(where) + ": " + buf);
  }
  return rc;
}

// Dense row-major block with its non-zero count (the part of MatrixBlock this path needs).
struct MatrixBlock {
  int rlen = 0, clen = 0;
  int64_t nonZeros = -1;
  std::vector<double> values;
  MatrixBlock() {}
  MatrixBlock(int r, int c) : rlen(r), clen(c), values((size_t)r * c, 0.0) {}
  MatrixBlock(int r, int c, std::vector<double> v) : rlen(r), clen(c), values(std::move(v)) {}
  int getNumRows() const { return rlen; }
  int getNumColumns() const { return clen; }
  int64_t getNonZeros() const { return nonZeros; }
  double& at(int r, int c) { return values[(size_t)r * clen + c]; }
  double at(int r, int c) const { return values[(size_t)r * clen + c]; }
};

// AMapToData in the JVM's storage layout; MapToFactory::create picks the class by cardinality
// (colgroup/mapping/MapToFactory.java:102-117).
struct AMapToData {
  int type = CLA_MAP_ZERO;
  int64_t size = 0;
  int unique = 1;
  std::vector<uint8_t> data, hi;
  int getIndex(int64_t r) const {
    switch (type) {
      case CLA_MAP_ZERO: return 0;
      case CLA_MAP_BIT: return (int)((((const uint64_t*)data.data())[r >> 6] >> (r & 63)) & 1u);
      case CLA_MAP_UBYTE:
      case CLA_MAP_BYTE: return data[r];
      case CLA_MAP_CHAR: return ((const uint16_t*)data.data())[r];
      case CLA_MAP_CHAR_BYTE: return ((const uint16_t*)data.data())[r] + ((int)hi[r] << 16);
      default: return ((const int32_t*)data.data())[r];
    }
  }
};

struct MapToFactory {
  static int typeFor(int64_t size, int64_t unique) {
    if (unique <= 1) return CLA_MAP_ZERO;
    if (unique == 2 && size > 32) return CLA_MAP_BIT;
    if (unique <= 128) return CLA_MAP_UBYTE;
    if (unique <= 256) return CLA_MAP_BYTE;
    if (unique <= 65536) return CLA_MAP_CHAR;
    if (unique <= 8388608) return CLA_MAP_CHAR_BYTE;
    return CLA_MAP_INT;
  }
  static AMapToData create(const std::vector<int>& ids, int unique) {
    AMapToData m;
    m.size = (int64_t)ids.size();
    m.unique = unique;
    m.type = typeFor(m.size, unique);
    switch (m.type) {
      case CLA_MAP_ZERO: break;
      case CLA_MAP_BIT:
        m.data.assign((size_t)((m.size + 63) / 64) * 8, 0);
        for (int64_t r = 0; r < m.size; r++)
          if (ids[r]) ((uint64_t*)m.data.data())[r >> 6] |= 1ull << (r & 63);
        break;
      case CLA_MAP_UBYTE:
      case CLA_MAP_BYTE:
        m.data.resize(m.size);
        for (int64_t r = 0; r < m.size; r++) m.data[r] = (uint8_t)ids[r];
        break;
      case CLA_MAP_CHAR:
        m.data.resize(m.size * 2);
        for (int64_t r = 0; r < m.size; r++) ((uint16_t*)m.data.data())[r] = (uint16_t)ids[r];
        break;
      case CLA_MAP_CHAR_BYTE:
        m.data.resize(m.size * 2);
        m.hi.resize(m.size);
        for (int64_t r = 0; r < m.size; r++) {
          ((uint16_t*)m.data.data())[r] = (uint16_t)(ids[r] & 0xFFFF);
          m.hi[r] = (uint8_t)(ids[r] >> 16);
        }
        break;
      default:
        m.data.resize(m.size * 4);
        for (int64_t r = 0; r < m.size; r++) ((int32_t*)m.data.data())[r] = ids[r];
    }
    return m;
  }
};

// AOffset; OffsetFactory::createOffset restates colgroup/offset/OffsetFactory.java:105-149, :238-338.
struct AOffset {
  int type = CLA_OFF_EMPTY;
  int offsetToFirst = 0, offsetToLast = 0;
  int64_t size = 0;
  std::vector<uint8_t> data;  // u8 deltas (BYTE) or u16 deltas (CHAR)
  int64_t dataLen() const { return type == CLA_OFF_CHAR ? (int64_t)data.size() / 2 : (int64_t)data.size(); }
};

struct OffsetFactory {
  static double arrayCost(int64_t n, int width) {  // utils/MemoryEstimates.java:68-105
    double size = 8 + 20;
    const int64_t small = width == 1 ? 4 : 2;
    if (n <= small) return size + 4;
    size += (double)n * width;
    const double diff = (double)((n * width - 4) % 8);
    return size + (diff > 0 ? 8 - diff : 0);
  }
  static AOffset createOffset(const std::vector<int>& idx) {
    AOffset o;
    const int64_t n = (int64_t)idx.size();
    o.size = n;
    if (n == 0) return o;
    if (idx[0] < 0) throw DMLCompressionException(CLA_ERR_BAD_ARG, "Invalid negative offset");
    o.offsetToFirst = idx[0];
    o.offsetToLast = idx[n - 1];
    if (n == 1) { o.type = CLA_OFF_SINGLE; return o; }
    if (n == 2) { o.type = CLA_OFF_TWO; return o; }
    const int64_t endLength = n - 1, range = (int64_t)idx[n - 1] - idx[0];
    const int64_t corrB = std::max<int64_t>(range - endLength * 256, 0) / 256;
    const int64_t corrC = std::max<int64_t>(range - endLength * 65535, 0) / 65535;
    const int64_t byteSize = (int64_t)(16 + 4 + 4 + 4 + 8 + arrayCost(endLength + corrB, 1));
    const int64_t charSize = (int64_t)(16 + 4 + 4 + 8 + arrayCost(endLength + corrC, 2));
    const bool useByte = byteSize < charSize;
    const int maxV = useByte ? 255 : 65535;
    o.type = useByte ? CLA_OFF_BYTE : CLA_OFF_CHAR;
    std::vector<int> out;
    for (int64_t i = 1; i < n; i++) {
      const int gap = idx[i] - idx[i - 1];
      if (gap <= 0) throw DMLCompressionException(CLA_ERR_BAD_ARG, "Invalid input to create offset, all values should be continuously increasing");
      const int div = gap / maxV, mod = gap % maxV;
      for (int z = 0; z < (mod == 0 ? div - 1 : div); z++) out.push_back(0);
      out.push_back(mod == 0 ? maxV : mod);
    }
    if (useByte) {
      o.data.resize(out.size());
      for (size_t i = 0; i < out.size(); i++) o.data[i] = (uint8_t)out[i];
    } else {
      o.data.resize(out.size() * 2);
      for (size_t i = 0; i < out.size(); i++) ((uint16_t*)o.data.data())[i] = (uint16_t)out[i];
    }
    return o;
  }
};

// ---- column groups ------------------------------------------------------------------------------------
class AColGroup {
 public:
  std::vector<int32_t> _colIndexes;
  explicit AColGroup(std::vector<int32_t> cols) : _colIndexes(std::move(cols)) {}
  virtual ~AColGroup() {}
  int getNumCols() const { return (int)_colIndexes.size(); }
  virtual int getNumValues() const { return 0; }
  virtual int64_t registerWith(cla_handle h) const = 0;  // the matching cla_add_group_* call
};

class ADictBasedColGroup : public AColGroup {
 public:
  std::vector<double> _dict;  // [nVals x gCols] row-major (colgroup/dictionary/Dictionary.java:94-97)
  ADictBasedColGroup(std::vector<int32_t> cols, std::vector<double> dict) : AColGroup(std::move(cols)), _dict(std::move(dict)) {}
  int getNumValues() const override { return (int)(_dict.size() / _colIndexes.size()); }
};

class ColGroupDDC : public ADictBasedColGroup {
 public:
  AMapToData _data;
  ColGroupDDC(std::vector<int32_t> cols, std::vector<double> dict, AMapToData data)
      : ADictBasedColGroup(std::move(cols), std::move(dict)), _data(std::move(data)) {}
  int64_t registerWith(cla_handle h) const override {
    return cla_add_group_ddc(h, _colIndexes.data(), getNumCols(), _dict.data(), getNumValues(), _data.type,
                             _data.data.data(), _data.hi.empty() ? nullptr : _data.hi.data(), _data.size);
  }
};

// ColGroupSDC (default tuple), ColGroupSDCZeros (no default), and with no map the Single variants.
class ColGroupSDC : public ADictBasedColGroup {
 public:
  AOffset _indexes;
  std::unique_ptr<AMapToData> _data;     // null: SDCSingle / SDCSingleZeros
  std::vector<double> _defaultTuple;     // empty: *Zeros
  ColGroupSDC(std::vector<int32_t> cols, std::vector<double> dict, std::vector<double> defaultTuple, AOffset indexes,
              std::unique_ptr<AMapToData> data)
      : ADictBasedColGroup(std::move(cols), std::move(dict)), _indexes(std::move(indexes)), _data(std::move(data)),
        _defaultTuple(std::move(defaultTuple)) {}
  int64_t registerWith(cla_handle h) const override {
    static const int64_t dummy = 0;
    const void* mp = !_data ? nullptr : (_data->data.empty() ? (const void*)&dummy : (const void*)_data->data.data());
    return cla_add_group_sdc(h, _colIndexes.data(), getNumCols(), _dict.data(), getNumValues(),
                             _defaultTuple.empty() ? nullptr : _defaultTuple.data(), _indexes.type,
                             _indexes.offsetToFirst, _indexes.offsetToLast, _indexes.data.data(), _indexes.dataLen(),
                             _indexes.size, _data ? _data->type : 0, mp,
                             (_data && !_data->hi.empty()) ? _data->hi.data() : nullptr);
  }
};

class AColGroupOffset : public ADictBasedColGroup {
 public:
  std::vector<int32_t> _ptr;
  std::vector<uint16_t> _data;
  AColGroupOffset(std::vector<int32_t> cols, std::vector<double> dict, std::vector<int32_t> ptr, std::vector<uint16_t> data)
      : ADictBasedColGroup(std::move(cols), std::move(dict)), _ptr(std::move(ptr)), _data(std::move(data)) {}
};
class ColGroupRLE : public AColGroupOffset {
 public:
  using AColGroupOffset::AColGroupOffset;
  int64_t registerWith(cla_handle h) const override {
    return cla_add_group_rle(h, _colIndexes.data(), getNumCols(), _dict.data(), getNumValues(), _ptr.data(), _data.data(),
                             (int64_t)_data.size());
  }
};
class ColGroupOLE : public AColGroupOffset {
 public:
  using AColGroupOffset::AColGroupOffset;
  int64_t registerWith(cla_handle h) const override {
    return cla_add_group_ole(h, _colIndexes.data(), getNumCols(), _dict.data(), getNumValues(), _ptr.data(), _data.data(),
                             (int64_t)_data.size());
  }
};
class ColGroupUncompressed : public AColGroup {
 public:
  std::vector<double> _data;  // [nRows x gCols]
  ColGroupUncompressed(std::vector<int32_t> cols, std::vector<double> data) : AColGroup(std::move(cols)), _data(std::move(data)) {}
  int64_t registerWith(cla_handle h) const override {
    return cla_add_group_uncompressed(h, _colIndexes.data(), getNumCols(), _data.data());
  }
};
class ColGroupConst : public ADictBasedColGroup {
 public:
  using ADictBasedColGroup::ADictBasedColGroup;
  int64_t registerWith(cla_handle h) const override {
    return cla_add_group_const(h, _colIndexes.data(), getNumCols(), _dict.data());
  }
};
class ColGroupEmpty : public AColGroup {
 public:
  using AColGroup::AColGroup;
  int64_t registerWith(cla_handle h) const override { return cla_add_group_empty(h, _colIndexes.data(), getNumCols()); }
};

// ---- CompressedMatrixBlock (runtime/compress/CompressedMatrixBlock.java:108-132) -------------------------
class CompressedMatrixBlock {
  int rlen, clen;
  bool overlappingColGroups;
  std::vector<std::shared_ptr<AColGroup>> _colGroups;
  cla_handle handle_ = 0;

 public:
  CompressedMatrixBlock(int rl, int cl, bool overlapping = false) : rlen(rl), clen(cl), overlappingColGroups(overlapping) {}
  CompressedMatrixBlock(const CompressedMatrixBlock&) = delete;
  CompressedMatrixBlock& operator=(const CompressedMatrixBlock&) = delete;
  ~CompressedMatrixBlock() { if (handle_) cla_destroy(handle_); }
  int getNumRows() const { return rlen; }
  int getNumColumns() const { return clen; }
  bool isOverlapping() const { return overlappingColGroups; }
  const std::vector<std::shared_ptr<AColGroup>>& getColGroups() const { return _colGroups; }
  void allocateColGroup(std::shared_ptr<AColGroup> g) {
    if (handle_) throw DMLCompressionException(CLA_ERR_STATE, "block is already on the device");
    _colGroups.push_back(std::move(g));
  }
  // CompressedMatrixBlock.read(DataInput) (CompressedMatrixBlock.java:486-496): the serialized form goes to the
  // library's own reader and straight to the device; no host-side group objects are built.
  static std::unique_ptr<CompressedMatrixBlock> read(const uint8_t* bytes, int64_t len, int device = 0) {
    cla_handle h = check(cla_read_block(bytes, len, nullptr, nullptr), "cla_read_block");
    cla_stats st;
    try {
      check(cla_stats_get(h, &st), "cla_stats_get");
      check(cla_finalize(h, device), "cla_finalize");
    } catch (...) {
      cla_destroy(h);
      throw;
    }
    std::unique_ptr<CompressedMatrixBlock> b(new CompressedMatrixBlock((int)st.n_rows, (int)st.n_cols));
    b->handle_ = h;
    return b;
  }
  // wraps a handle the library returned (an overlapping product): already on the device, no host-side groups
  static std::unique_ptr<CompressedMatrixBlock> adopt(cla_handle h, int rows, int cols) {
    std::unique_ptr<CompressedMatrixBlock> b(new CompressedMatrixBlock(rows, cols, true));
    b->handle_ = h;
    return b;
  }
  // uploads the groups on first use (cla_create .. cla_finalize)
  cla_handle nativeHandle(int device = 0) {
    if (!handle_) {
      cla_handle h = check(cla_create(rlen, clen, overlappingColGroups ? 1 : 0), "cla_create");
      try {
        for (auto& g : _colGroups) check(g->registerWith(h), "cla_add_group");
        check(cla_finalize(h, device), "cla_finalize");
      } catch (...) {
        cla_destroy(h);
        throw;
      }
      handle_ = h;
    }
    return handle_;
  }
};

// ---- the CLALib entry points ---------------------------------------------------------------------------
struct CLALibRightMultBy {  // lib/CLALibRightMultBy.java:57
  static MatrixBlock rightMultByMatrix(CompressedMatrixBlock& m1, const MatrixBlock& m2) {
    MatrixBlock ret(m1.getNumRows(), m2.clen);
    try {
      ret.nonZeros = check(cla_rmm(m1.nativeHandle(), m2.values.data(), m2.rlen, m2.clen, ret.values.data()), "cla_rmm");
    } catch (const DMLCompressionException& e) {
      throw DMLCompressionException(e.code, std::string("Failed Right MM: ") + e.what());  // :99-101
    }
    return ret;
  }
  // allowOverlap = true (lib/CLALibRightMultBy.java:61-64, RMMOverlapping :127-161): the product stays compressed, an
  // overlapping block on the device that shares m1's index structures (m1 must outlive it or be destroyed first:
  // the library keeps what the result still needs)
  static std::unique_ptr<CompressedMatrixBlock> rightMultByMatrixOverlapping(CompressedMatrixBlock& m1, const MatrixBlock& m2) {
    cla_handle h = check(cla_rmm_overlapping(m1.nativeHandle(), m2.values.data(), m2.rlen, m2.clen), "cla_rmm_overlapping");
    return CompressedMatrixBlock::adopt(h, m1.getNumRows(), m2.clen);
  }
};
struct CLALibLeftMultBy {  // lib/CLALibLeftMultBy.java:126; left is [q x nRows]
  static MatrixBlock leftMultByMatrix(CompressedMatrixBlock& right, const MatrixBlock& left) {
    if (left.clen != right.getNumRows()) throw DMLCompressionException(CLA_ERR_SHAPE, "Failed CLA LMM: inner dimensions differ");
    MatrixBlock ret(left.rlen, right.getNumColumns());
    try {
      ret.nonZeros = check(cla_lmm(right.nativeHandle(), left.values.data(), left.rlen, ret.values.data()), "cla_lmm");
    } catch (const DMLCompressionException& e) {
      throw DMLCompressionException(e.code, std::string("Failed CLA LMM: ") + e.what());  // :142-144
    }
    return ret;
  }
};
struct CLALibLeftMultByCompressed {  // lib/CLALibLeftMultBy.java:100: t(left) %*% right, both compressed
  static MatrixBlock leftMultByMatrixTransposed(CompressedMatrixBlock& right, CompressedMatrixBlock& left) {
    if (left.getNumRows() != right.getNumRows())
      throw DMLCompressionException(CLA_ERR_SHAPE, "Failed CLA Compressed Transposed LMM: row counts differ");
    MatrixBlock ret(left.getNumColumns(), right.getNumColumns());
    try {
      ret.nonZeros = check(cla_tmm(left.nativeHandle(), right.nativeHandle(), ret.values.data()), "cla_tmm");
    } catch (const DMLCompressionException& e) {
      throw DMLCompressionException(e.code, std::string("Failed CLA Compressed Transposed LMM: ") + e.what());  // :109-111
    }
    return ret;
  }
};
struct CLALibTSMM {  // lib/CLALibTSMM.java:59
  static MatrixBlock leftMultByTransposeSelf(CompressedMatrixBlock& cmb) {
    MatrixBlock ret(cmb.getNumColumns(), cmb.getNumColumns());
    ret.nonZeros = check(cla_tsmm(cmb.nativeHandle(), ret.values.data()), "cla_tsmm");
    return ret;
  }
};
struct CLALibMMChain {  // lib/CLALibMMChain.java:92; w may be null for XtXv
  static MatrixBlock mmChain(CompressedMatrixBlock& x, const MatrixBlock& v, const MatrixBlock* w, int ctype) {
    if ((int)v.values.size() != x.getNumColumns()) throw DMLCompressionException(CLA_ERR_SHAPE, "mmChain: v must have nCols entries");
    MatrixBlock ret(x.getNumColumns(), 1);
    ret.nonZeros = check(cla_mmchain(x.nativeHandle(), v.values.data(), w ? w->values.data() : nullptr, ctype, ret.values.data()), "cla_mmchain");
    return ret;
  }
};
struct CLALibCompAgg {  // lib/CLALibCompAgg.java: uack+ / uark+ / uak+ and the min / max cases
  static MatrixBlock aggregate(CompressedMatrixBlock& cmb, int op) {
    const bool col = op == CLA_AGG_COL_SUMS || op == CLA_AGG_COL_MINS || op == CLA_AGG_COL_MAXS;
    const bool row = op == CLA_AGG_ROW_SUMS || op == CLA_AGG_ROW_MINS || op == CLA_AGG_ROW_MAXS;
    MatrixBlock ret(row ? cmb.getNumRows() : 1, col ? cmb.getNumColumns() : 1);
    ret.nonZeros = check(cla_unary_agg(cmb.nativeHandle(), op, ret.values.data()), "cla_unary_agg");
    return ret;
  }
  static MatrixBlock colSums(CompressedMatrixBlock& c) { return aggregate(c, CLA_AGG_COL_SUMS); }
  static MatrixBlock rowSums(CompressedMatrixBlock& c) { return aggregate(c, CLA_AGG_ROW_SUMS); }
  static MatrixBlock colMins(CompressedMatrixBlock& c) { return aggregate(c, CLA_AGG_COL_MINS); }
  static MatrixBlock colMaxs(CompressedMatrixBlock& c) { return aggregate(c, CLA_AGG_COL_MAXS); }
  static MatrixBlock rowMins(CompressedMatrixBlock& c) { return aggregate(c, CLA_AGG_ROW_MINS); }
  static MatrixBlock rowMaxs(CompressedMatrixBlock& c) { return aggregate(c, CLA_AGG_ROW_MAXS); }
  static double sum(CompressedMatrixBlock& c) { return aggregate(c, CLA_AGG_SUM).values[0]; }
  static double min(CompressedMatrixBlock& c) { return aggregate(c, CLA_AGG_MIN).values[0]; }
  static double max(CompressedMatrixBlock& c) { return aggregate(c, CLA_AGG_MAX).values[0]; }
};
struct CLALibDecompress {  // lib/CLALibDecompress.java:56
  static MatrixBlock decompress(CompressedMatrixBlock& cmb) {
    MatrixBlock ret(cmb.getNumRows(), cmb.getNumColumns());
    ret.nonZeros = check(cla_decompress(cmb.nativeHandle(), ret.values.data()), "cla_decompress");
    return ret;
  }
};

// The sum over row shards on the GPUs of one node (one process per GPU), over NVLink peer memory; no counterpart in
// the reference. exchange(mine, all) must fill `all` with the CLA_COMM_HANDLE_BYTES-byte handles of all ranks in rank
// order (MPI_Allgather or whatever the host uses).
class PeerAllReduce {
  int64_t comm_ = 0;

 public:
  template <class Exchange>
  PeerAllReduce(int device, int rank, int world, int64_t maxDoubles, Exchange&& exchange) {
    std::vector<char> mine(CLA_COMM_HANDLE_BYTES), all((size_t)world * CLA_COMM_HANDLE_BYTES);
    comm_ = check(cla_comm_create(device, rank, world, maxDoubles, mine.data()), "cla_comm_create");
    try {
      exchange(mine.data(), all.data());
      check(cla_comm_connect(comm_, all.data()), "cla_comm_connect");
    } catch (...) {
      cla_comm_destroy(comm_);
      throw;
    }
  }
  PeerAllReduce(const PeerAllReduce&) = delete;
  PeerAllReduce& operator=(const PeerAllReduce&) = delete;
  ~PeerAllReduce() { if (comm_) cla_comm_destroy(comm_); }
  // in place on a device buffer, enqueued on `stream`; every rank ends with identical bits
  void operator()(double* dBuf, int64_t n, void* stream) { check(cla_allreduce_dev(comm_, dBuf, n, stream), "cla_allreduce_dev"); }
  void status() { check(cla_comm_status(comm_), "cla_comm_status"); }  // throws if a rank failed to arrive earlier
};


}  // namespace cla
}  // namespace sysds
