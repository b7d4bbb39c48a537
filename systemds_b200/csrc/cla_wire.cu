// Reader for the serialized form of a CompressedMatrixBlock: the byte stream the reference writes with
// CompressedMatrixBlock.write(DataOutput) (runtime/compress/CompressedMatrixBlock.java:497-519) and reads back with
// read(DataInput) (:486-496), i.e. what a Spark broadcast, a buffer-pool eviction or a binary file holds. The stream
// is big-endian (java.io.DataOutput). Every group is registered through the same cla_add_group_* calls a host would
// make itself, so all their validation applies; the handle comes back open (not finalized).
//
// Layout, field by field (colgroup/ColGroupIO.java:48-139 and the write() of each class):
//   block : int rlen, int clen, long nonZeros, boolean overlapping, int nGroups, groups
//   group : byte ColGroupType ordinal (colgroup/AColGroup.java:89-92), column index, class payload
//   index : byte ColIndexType ordinal (colgroup/indexes/IColIndex.java:33-35): SINGLE int | TWO int int |
//           ARRAY int n, int[n] | RANGE int l, int u | TWORANGE int l1, int n1, int l2, int n2 | COMBINED index index
//   dict  : byte DictionaryFactory.Type ordinal (colgroup/dictionary/DictionaryFactory.java:54-77):
//           FP64 int n, double[n] | MATRIX_BLOCK MatrixBlock | IDENTITY int n; the others are refused
//   map   : byte MAP_TYPE ordinal; ZERO int size | BIT int size, int words, long[words] |
//           UBYTE/BYTE int unique, int n, byte[n] | CHAR int unique, int n, char[n] |
//           CHAR_BYTE int unique, int n, char[n], byte[n] | INT int unique, int n, int[n]  (colgroup/mapping/Map*.java)
//   offset: byte OFF_TYPE_SPECIALIZATIONS ordinal (colgroup/offset/OffsetFactory.java:46-52):
//           BYTE int first, int n, int last, int size, byte[n] | BYTENZ/BYTEUNZ int first, int n, int last, byte[n] |
//           CHAR int first, int n, int last, char[n] | SINGLE int | TWO int int | EMPTY
//   MatrixBlock (runtime/matrix/data/MatrixBlock.java:2111-2165): int rlen, int clen, byte BlockType;
//           EMPTY | DENSE double[rlen*clen] | SPARSE nnz (long if rlen*clen > Integer.MAX_VALUE else int), per row
//           int n, (int col, double v)[n] | ULTRA_SPARSE int nnz, (int row, int col, double v)[nnz] or, with one
//           column, (int row, double v)[nnz]
#include "../../include/systemds_cla.h"
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace cla {
int64_t fail(int64_t code, const std::string& msg);
}

namespace {

struct Truncated : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct Unsupported : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct In {
  const uint8_t* b;
  int64_t n, p = 0;
  const uint8_t* take(int64_t k) {
    if (k < 0 || p + k > n) throw Truncated("the stream ends inside a field at offset " + std::to_string(p));
    const uint8_t* r = b + p;
    p += k;
    return r;
  }
  int u8() { return *take(1); }
  int32_t i32() {
    const uint8_t* q = take(4);
    return (int32_t)(((uint32_t)q[0] << 24) | ((uint32_t)q[1] << 16) | ((uint32_t)q[2] << 8) | (uint32_t)q[3]);
  }
  int64_t i64() {
    const uint64_t hi = (uint32_t)i32();
    const uint64_t lo = (uint32_t)i32();
    return (int64_t)((hi << 32) | lo);
  }
  double f64() {
    const int64_t v = i64();
    double d;
    std::memcpy(&d, &v, 8);
    return d;
  }
  int32_t len() {
    const int32_t v = i32();
    if (v < 0) throw Truncated("negative array length at offset " + std::to_string(p - 4));
    return v;
  }
  void bytes(std::vector<uint8_t>& out, int64_t k) {
    const uint8_t* q = take(k);
    out.assign(q, q + k);
  }
  void u16s(std::vector<uint16_t>& out, int64_t k) {
    const uint8_t* q = take(2 * k);
    out.resize(k);
    for (int64_t i = 0; i < k; i++) out[i] = (uint16_t)((q[2 * i] << 8) | q[2 * i + 1]);
  }
  void i32s(std::vector<int32_t>& out, int64_t k) {
    const uint8_t* q = take(4 * k);
    out.resize(k);
    for (int64_t i = 0; i < k; i++)
      out[i] = (int32_t)(((uint32_t)q[4 * i] << 24) | ((uint32_t)q[4 * i + 1] << 16) | ((uint32_t)q[4 * i + 2] << 8) | (uint32_t)q[4 * i + 3]);
  }
  void f64s(std::vector<double>& out, int64_t k) {
    const uint8_t* q = take(8 * k);
    out.resize(k);
    for (int64_t i = 0; i < k; i++) {
      uint64_t v = 0;
      for (int j = 0; j < 8; j++) v = (v << 8) | q[8 * i + j];
      std::memcpy(&out[i], &v, 8);
    }
  }
};

void read_index(In& s, std::vector<int32_t>& cols) {
  const int t = s.u8();
  switch (t) {
    case 0: cols.push_back(s.i32()); break;
    case 1: cols.push_back(s.i32()); cols.push_back(s.i32()); break;
    case 2: {
      const int32_t n = s.len();
      for (int32_t i = 0; i < n; i++) cols.push_back(s.i32());
      break;
    }
    case 3: {
      const int32_t l = s.i32(), u = s.i32();
      for (int32_t c = l; c < u; c++) cols.push_back(c);
      break;
    }
    case 4: {
      const int32_t l1 = s.i32(), n1 = s.i32(), l2 = s.i32(), n2 = s.i32();
      for (int32_t c = 0; c < n1; c++) cols.push_back(l1 + c);
      for (int32_t c = 0; c < n2; c++) cols.push_back(l2 + c);
      break;
    }
    case 5: read_index(s, cols); read_index(s, cols); break;  // left then right (CombinedIndex.get)
    default: throw Unsupported("unknown column index type " + std::to_string(t));
  }
}

// dense row-major [rlen x clen]
void read_matrix_block(In& s, std::vector<double>& out, int32_t& rlen, int32_t& clen) {
  rlen = s.len();
  clen = s.len();
  const int fmt = s.u8();
  const int64_t cells = (int64_t)rlen * clen;
  if (fmt == 3) {  // DENSE_BLOCK
    s.f64s(out, cells);
    return;
  }
  if (fmt == 4) throw Unsupported("de-duplicated dense blocks are not supported");
  if (fmt > 4) throw Unsupported("unknown block format " + std::to_string(fmt));
  // a corrupted length must not allocate without bound: an empty block may be large (it needs no bytes), the
  // sparse formats must be accounted for by what is left of the stream
  if (cells > (fmt == 0 ? (int64_t)1 << 28 : (int64_t)s.n * 64)) throw Truncated("block dimensions exceed what the stream can hold");
  out.assign((size_t)cells, 0.0);
  if (fmt == 0) return;  // EMPTY_BLOCK
  if (fmt == 2) {        // SPARSE_BLOCK
    if (cells > 2147483647ll) s.i64(); else s.i32();
    for (int32_t r = 0; r < rlen; r++) {
      const int32_t k = s.len();
      for (int32_t j = 0; j < k; j++) {
        const int32_t c = s.i32();
        const double v = s.f64();
        if (c < 0 || c >= clen) throw Unsupported("sparse block: column index outside the block");
        out[(size_t)r * clen + c] = v;
      }
    }
    return;
  }
  const int32_t nnz = s.len();  // ULTRA_SPARSE_BLOCK
  for (int32_t i = 0; i < nnz; i++) {
    const int32_t r = s.i32();
    const int32_t c = clen > 1 ? s.i32() : 0;
    const double v = s.f64();
    if (r < 0 || r >= rlen || c < 0 || c >= clen) throw Unsupported("ultra-sparse block: cell outside the block");
    out[(size_t)r * clen + c] = v;
  }
}

void read_dict(In& s, int gCols, std::vector<double>& d, int32_t& nVals) {
  const int t = s.u8();
  if (t == 0) {  // FP64_DICT
    const int32_t n = s.len();
    if (gCols == 0 || n % gCols) throw Unsupported("dictionary size is not a multiple of the group's column count");
    s.f64s(d, n);
    nVals = n / gCols;
  } else if (t == 1) {  // MATRIX_BLOCK_DICT
    int32_t r, c;
    read_matrix_block(s, d, r, c);
    if (c != gCols) throw Unsupported("matrix-block dictionary width differs from the group's column count");
    nVals = r;
  } else if (t == 3) {  // IDENTITY
    const int32_t n = s.len();
    if (n != gCols) throw Unsupported("identity dictionary width differs from the group's column count");
    d.assign((size_t)n * n, 0.0);
    for (int32_t i = 0; i < n; i++) d[(size_t)i * n + i] = 1.0;
    nVals = n;
  } else
    throw Unsupported("dictionary type ordinal " + std::to_string(t) + " is not supported");
}

struct Map {
  int32_t type = CLA_MAP_ZERO;
  int64_t size = 0;
  std::vector<uint8_t> b;    // UBYTE / BYTE, or the byte plane of CHAR_BYTE
  std::vector<uint16_t> c;   // CHAR / CHAR_BYTE
  std::vector<int32_t> i;    // INT
  std::vector<uint64_t> w;   // BIT
  const void* lo() const {
    switch (type) {
      case CLA_MAP_BIT: return w.data();
      case CLA_MAP_UBYTE:
      case CLA_MAP_BYTE: return b.data();
      case CLA_MAP_CHAR:
      case CLA_MAP_CHAR_BYTE: return c.data();
      case CLA_MAP_INT: return i.data();
      default: return nullptr;
    }
  }
  const void* hi() const { return type == CLA_MAP_CHAR_BYTE ? b.data() : nullptr; }
};

void read_map(In& s, Map& m) {
  m.type = s.u8();
  switch (m.type) {
    case CLA_MAP_ZERO: m.size = s.len(); break;
    case CLA_MAP_BIT: {
      m.size = s.len();
      const int32_t words = s.len();
      m.w.resize(words);
      for (int32_t k = 0; k < words; k++) m.w[k] = (uint64_t)s.i64();
      if ((int64_t)words * 64 < m.size) throw Unsupported("bit map holds fewer words than its size needs");
      break;
    }
    case CLA_MAP_UBYTE:
    case CLA_MAP_BYTE: s.i32(); m.size = s.len(); s.bytes(m.b, m.size); break;
    case CLA_MAP_CHAR: s.i32(); m.size = s.len(); s.u16s(m.c, m.size); break;
    case CLA_MAP_CHAR_BYTE: s.i32(); m.size = s.len(); s.u16s(m.c, m.size); s.bytes(m.b, m.size); break;
    case CLA_MAP_INT: s.i32(); m.size = s.len(); s.i32s(m.i, m.size); break;
    default: throw Unsupported("unknown map type " + std::to_string(m.type));
  }
}

struct Off {
  int32_t type = CLA_OFF_EMPTY, first = 0, last = 0;
  int64_t size = 0, len = 0;
  std::vector<uint8_t> b;
  std::vector<uint16_t> c;
  const void* data() const { return type == CLA_OFF_BYTE ? (const void*)b.data() : (type == CLA_OFF_CHAR ? (const void*)c.data() : nullptr); }
};

void read_offsets(In& s, Off& o) {
  const int t = s.u8();
  switch (t) {
    case 4: o.type = CLA_OFF_EMPTY; break;
    case 2: o.type = CLA_OFF_SINGLE; o.first = o.last = s.i32(); o.size = 1; break;
    case 3: o.type = CLA_OFF_TWO; o.first = s.i32(); o.last = s.i32(); o.size = 2; break;
    case 0: case 5: case 6: {  // BYTE, BYTEUNZ, BYTENZ
      o.type = CLA_OFF_BYTE;
      o.first = s.i32();
      o.len = s.len();
      o.last = s.i32();
      o.size = t == 0 ? (int64_t)s.len() : o.len + 1;
      s.bytes(o.b, o.len);
      break;
    }
    case 1: {  // CHAR: the size is one more than the number of non-zero deltas (OffsetChar.java:123-134)
      o.type = CLA_OFF_CHAR;
      o.first = s.i32();
      o.len = s.len();
      o.last = s.i32();
      s.u16s(o.c, o.len);
      o.size = 1;
      for (uint16_t v : o.c) o.size += v != 0;
      break;
    }
    default: throw Unsupported("unknown offset type " + std::to_string(t));
  }
}

struct Status {  // a failed cla_add_group_* call: its message is already recorded
  int64_t code;
};
inline void ok(int64_t rc) {
  if (rc < 0) throw Status{rc};
}

void read_group(In& s, cla_handle h, int32_t nRows) {
  const int t = s.u8();
  std::vector<int32_t> cols;
  read_index(s, cols);
  const int gc = (int)cols.size();
  std::vector<double> dict, tuple;
  int32_t nVals = 0;
  Map map;
  Off off;
  switch (t) {
    case 5: ok(cla_add_group_empty(h, cols.data(), gc)); return;
    case 0: {  // UNCOMPRESSED
      int32_t r, c;
      read_matrix_block(s, dict, r, c);
      if (r != nRows || c != gc) throw Unsupported("uncompressed group: block shape differs from the group's");
      ok(cla_add_group_uncompressed(h, cols.data(), gc, dict.data()));
      return;
    }
    case 12: case 13: case 14:
      throw Unsupported("column group type ordinal " + std::to_string(t) + " (LZW / delta / linear functional) is not supported");
    default:
      if (t > 14) throw Unsupported("unknown column group type " + std::to_string(t));
  }
  read_dict(s, gc, dict, nVals);
  switch (t) {
    case 4:  // CONST
      if (nVals != 1) throw Unsupported("constant group with more than one tuple");
      ok(cla_add_group_const(h, cols.data(), gc, dict.data()));
      return;
    case 3: case 11:  // DDC, DDCFOR (value = dict[id] + reference: the reference tuple becomes a constant group)
      read_map(s, map);
      ok(cla_add_group_ddc(h, cols.data(), gc, dict.data(), nVals, map.type, map.lo(), map.hi(), map.size));
      if (t == 11) {
        s.f64s(tuple, gc);
        ok(cla_add_group_const(h, cols.data(), gc, tuple.data()));
      }
      return;
    case 1: case 2: {  // RLE, OLE
      std::vector<int32_t> ptr;
      std::vector<uint16_t> data;
      const int32_t np = s.len();
      s.i32s(ptr, np);
      const int32_t nd = s.len();
      s.u16s(data, nd);
      s.u8();  // _zeros: implied by the runs
      if (np != nVals + 1) throw Unsupported("offset group: _ptr must have nVals + 1 entries");
      ok((t == 1 ? cla_add_group_rle : cla_add_group_ole)(h, cols.data(), gc, dict.data(), nVals, ptr.data(), data.data(), nd));
      return;
    }
    default: break;
  }
  read_offsets(s, off);
  const bool hasMap = (t == 6 || t == 9 || t == 10);  // SDC, SDCZeros, SDCFOR
  if (hasMap) read_map(s, map);
  const bool hasDefault = (t == 6 || t == 7);          // SDC, SDCSingle
  if (hasDefault || t == 10) s.f64s(tuple, gc);
  ok(cla_add_group_sdc(h, cols.data(), gc, dict.data(), nVals, hasDefault ? tuple.data() : nullptr, off.type, off.first,
                       off.last, off.data(), off.len, off.size, hasMap ? map.type : CLA_MAP_ZERO,
                       hasMap ? map.lo() : nullptr, hasMap ? map.hi() : nullptr));
  if (t == 10) ok(cla_add_group_const(h, cols.data(), gc, tuple.data()));  // SDCFOR: + reference on every row
}

}  // namespace

extern "C" cla_handle cla_read_block(const uint8_t* bytes, int64_t len, int64_t* nonZeros, int64_t* consumed) {
  if (!bytes || len < 0) return cla::fail(CLA_ERR_BAD_ARG, "read_block: null buffer");
  In s{bytes, len};
  cla_handle h = 0;
  try {
    const int32_t rlen = s.i32(), clen = s.i32();
    const int64_t nnz = s.i64();
    const int overlapping = s.u8();
    const int32_t nGroups = s.len();
    if (rlen < 0 || clen < 0) return cla::fail(CLA_ERR_SHAPE, "read_block: negative dimension in the header");
    h = cla_create(rlen, clen, overlapping != 0);
    if (h < 0) return h;
    for (int32_t g = 0; g < nGroups; g++) read_group(s, h, rlen);
    if (nonZeros) *nonZeros = nnz;
    if (consumed) *consumed = s.p;
    return h;
  } catch (const Status& e) {
    if (h > 0) cla_destroy(h);
    return e.code;
  } catch (const Truncated& e) {
    if (h > 0) cla_destroy(h);
    return cla::fail(CLA_ERR_BAD_ARG, std::string("read_block: ") + e.what());
  } catch (const Unsupported& e) {
    if (h > 0) cla_destroy(h);
    return cla::fail(CLA_ERR_UNSUPPORTED, std::string("read_block: ") + e.what());
  } catch (const std::bad_alloc&) {
    if (h > 0) cla_destroy(h);
    return cla::fail(CLA_ERR_NOMEM, "read_block: out of host memory");
  }
}
