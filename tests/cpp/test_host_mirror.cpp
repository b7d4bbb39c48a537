// Builds a small CompressedMatrixBlock through the C++ host mirror (include/systemds_cla.hpp), runs every product on
// the GPU and compares with a plain dense evaluation of the same matrix. Exit codes: 0 ok, 1 mismatch,
// 3 no usable GPU (the library has no CPU path and says so), 2 any other failure.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <random>
#include "../../include/systemds_cla.hpp"

using namespace sysds::cla;

static double relErr(const std::vector<double>& got, const std::vector<double>& ref, const std::vector<double>& scale) {
  double e = 0;
  for (size_t i = 0; i < ref.size(); i++) e = std::max(e, std::fabs(got[i] - ref[i]) / std::max(scale[i], 1e-300));
  return e;
}

int main() {
  const int n = 9000, m = 6;
  std::mt19937_64 rng(42);
  std::normal_distribution<double> N(0, 1);
  std::vector<double> X((size_t)n * m, 0.0);
  CompressedMatrixBlock cmb(n, m);
  {  // DDC, two co-coded columns, 37 tuples (MapToUByte)
    std::vector<double> dict(37 * 2);
    for (auto& d : dict) d = N(rng);
    std::vector<int> ids(n);
    for (int r = 0; r < n; r++) {
      ids[r] = (int)(rng() % 37);
      X[(size_t)r * m + 0] = dict[ids[r] * 2];
      X[(size_t)r * m + 1] = dict[ids[r] * 2 + 1];
    }
    cmb.allocateColGroup(std::make_shared<ColGroupDDC>(std::vector<int32_t>{0, 1}, dict, MapToFactory::create(ids, 37)));
  }
  {  // DDC on a bit map
    std::vector<double> dict{N(rng), N(rng)};
    std::vector<int> ids(n);
    for (int r = 0; r < n; r++) {
      ids[r] = (int)(rng() & 1);
      X[(size_t)r * m + 2] = dict[ids[r]];
    }
    cmb.allocateColGroup(std::make_shared<ColGroupDDC>(std::vector<int32_t>{2}, dict, MapToFactory::create(ids, 2)));
  }
  {  // SDC with a non-zero default: every ~23rd row listed, long gaps in between to exercise continuation deltas
    std::vector<double> dict{N(rng), N(rng), N(rng)};
    const double def = 0.5;
    std::vector<int> rows, ids;
    for (int r = 3; r < n; r += 1 + (int)(rng() % 45) + ((rng() % 17 == 0) ? 700 : 0)) {
      rows.push_back(r);
      ids.push_back((int)(rng() % 3));
    }
    for (int r = 0; r < n; r++) X[(size_t)r * m + 3] = def;
    for (size_t i = 0; i < rows.size(); i++) X[(size_t)rows[i] * m + 3] = dict[ids[i]];
    cmb.allocateColGroup(std::make_shared<ColGroupSDC>(std::vector<int32_t>{3}, dict, std::vector<double>{def},
                                                       OffsetFactory::createOffset(rows),
                                                       std::make_unique<AMapToData>(MapToFactory::create(ids, 3))));
  }
  {  // RLE: value 0 on rows [10, 4000), value 1 on rows [4000, 4100) and [8000, 9000); (gap, len) pairs
    std::vector<double> dict{N(rng), N(rng)};
    std::vector<uint16_t> data{10, 3990, /* value 1: */ 4000, 100, 3900, 1000};
    std::vector<int32_t> ptr{0, 2, 6};
    for (int r = 10; r < 4000; r++) X[(size_t)r * m + 4] = dict[0];
    for (int r = 4000; r < 4100; r++) X[(size_t)r * m + 4] = dict[1];
    for (int r = 8000; r < 9000; r++) X[(size_t)r * m + 4] = dict[1];
    cmb.allocateColGroup(std::make_shared<ColGroupRLE>(std::vector<int32_t>{4}, dict, ptr, data));
  }
  cmb.allocateColGroup(std::make_shared<ColGroupConst>(std::vector<int32_t>{5}, std::vector<double>{-2.25}));
  for (int r = 0; r < n; r++) X[(size_t)r * m + 5] = -2.25;

  try {
    MatrixBlock V(m, 3), Yt(2, n), v(m, 1);
    for (auto& x : V.values) x = N(rng);
    for (auto& x : Yt.values) x = N(rng);
    for (auto& x : v.values) x = N(rng);
    int bad = 0;
    auto report = [&](const char* what, double e, double tol) {
      std::printf("%-12s rel err %.2e %s\n", what, e, e < tol ? "ok" : "MISMATCH");
      bad += !(e < tol);
    };
    {  // decompress
      MatrixBlock D = CLALibDecompress::decompress(cmb);
      std::vector<double> sc(X.size());
      for (size_t i = 0; i < X.size(); i++) sc[i] = std::max(std::fabs(X[i]), 1.0);
      report("decompress", relErr(D.values, X, sc), 1e-14);
    }
    {  // X %*% V
      MatrixBlock R = CLALibRightMultBy::rightMultByMatrix(cmb, V);
      std::vector<double> ref((size_t)n * 3, 0.0), sc((size_t)n * 3, 0.0);
      for (int r = 0; r < n; r++)
        for (int c = 0; c < m; c++)
          for (int j = 0; j < 3; j++) {
            ref[(size_t)r * 3 + j] += X[(size_t)r * m + c] * V.at(c, j);
            sc[(size_t)r * 3 + j] += std::fabs(X[(size_t)r * m + c] * V.at(c, j));
          }
      report("rmm", relErr(R.values, ref, sc), 1e-12);
      int64_t nnz = 0;
      for (double x : R.values) nnz += x != 0.0;
      if (nnz != R.getNonZeros()) { std::printf("nnz %lld != %lld\n", (long long)R.getNonZeros(), (long long)nnz); bad++; }
      // the same product kept compressed (allowOverlap): its decompressed form is the dense product
      std::unique_ptr<CompressedMatrixBlock> RO = CLALibRightMultBy::rightMultByMatrixOverlapping(cmb, V);
      MatrixBlock D = CLALibDecompress::decompress(*RO);
      report("rmm overlapping", relErr(D.values, ref, sc), 1e-12);
    }
    {  // Yt %*% X
      MatrixBlock L = CLALibLeftMultBy::leftMultByMatrix(cmb, Yt);
      std::vector<double> ref(2 * m, 0.0), sc(2 * m, 0.0);
      for (int i = 0; i < 2; i++)
        for (int r = 0; r < n; r++)
          for (int c = 0; c < m; c++) {
            ref[i * m + c] += Yt.at(i, r) * X[(size_t)r * m + c];
            sc[i * m + c] += std::fabs(Yt.at(i, r) * X[(size_t)r * m + c]);
          }
      report("lmm", relErr(L.values, ref, sc), 1e-12);
    }
    {  // t(X) %*% X and the chain
      MatrixBlock T = CLALibTSMM::leftMultByTransposeSelf(cmb);
      std::vector<double> ref(m * m, 0.0), sc(m * m, 0.0);
      for (int r = 0; r < n; r++)
        for (int a = 0; a < m; a++)
          for (int b = 0; b < m; b++) {
            ref[a * m + b] += X[(size_t)r * m + a] * X[(size_t)r * m + b];
            sc[a * m + b] += std::fabs(X[(size_t)r * m + a] * X[(size_t)r * m + b]);
          }
      report("tsmm", relErr(T.values, ref, sc), 1e-12);
      MatrixBlock W = CLALibMMChain::mmChain(cmb, v, nullptr, CLA_CHAIN_XtXv);
      std::vector<double> refw(m, 0.0), scw(m, 0.0);
      for (int a = 0; a < m; a++)
        for (int b = 0; b < m; b++) {
          refw[a] += ref[a * m + b] * v.values[b];
          scw[a] += sc[a * m + b] * std::fabs(v.values[b]);
        }
      report("mmchain", relErr(W.values, refw, scw), 1e-11);
    }
    {  // t(B) %*% X with B a second compressed block over the same rows (two dense columns)
      std::vector<double> Bv((size_t)n * 2);
      for (auto& x : Bv) x = N(rng);
      CompressedMatrixBlock B(n, 2);
      B.allocateColGroup(std::make_shared<ColGroupUncompressed>(std::vector<int32_t>{0, 1}, Bv));
      MatrixBlock T = CLALibLeftMultByCompressed::leftMultByMatrixTransposed(cmb, B);
      std::vector<double> ref(2 * m, 0.0), sc(2 * m, 0.0);
      for (int r = 0; r < n; r++)
        for (int a = 0; a < 2; a++)
          for (int b = 0; b < m; b++) {
            ref[a * m + b] += Bv[(size_t)r * 2 + a] * X[(size_t)r * m + b];
            sc[a * m + b] += std::fabs(Bv[(size_t)r * 2 + a] * X[(size_t)r * m + b]);
          }
      report("tmm", relErr(T.values, ref, sc), 1e-12);
    }
    {  // aggregates: column sums against the dense matrix, extrema bracket it
      MatrixBlock cs = CLALibCompAgg::colSums(cmb), lo = CLALibCompAgg::colMins(cmb), hi = CLALibCompAgg::colMaxs(cmb);
      std::vector<double> ref(m, 0.0), sc(m, 0.0);
      bool bracket = true;
      for (int r = 0; r < n; r++)
        for (int c = 0; c < m; c++) {
          ref[c] += X[(size_t)r * m + c];
          sc[c] += std::fabs(X[(size_t)r * m + c]);
          bracket &= lo.values[c] <= X[(size_t)r * m + c] && X[(size_t)r * m + c] <= hi.values[c];
        }
      report("colSums", relErr(cs.values, ref, sc), 1e-12);
      if (!bracket || !(CLALibCompAgg::min(cmb) <= CLALibCompAgg::max(cmb))) { std::printf("min/max do not bracket the data\n"); bad++; }
    }
    {  // error behaviour: shape mismatch surfaces as the reference's exception with its message prefix
      bool thrown = false;
      try {
        CLALibLeftMultBy::leftMultByMatrix(cmb, MatrixBlock(1, n - 1));
      } catch (const DMLCompressionException& e) {
        thrown = std::string(e.what()).find("Failed CLA LMM") == 0 && e.code == CLA_ERR_SHAPE;
      }
      if (!thrown) { std::printf("shape mismatch not reported\n"); bad++; }
    }
    return bad ? 1 : 0;
  } catch (const DMLCompressionException& e) {
    std::printf("DMLCompressionException(%lld): %s\n", (long long)e.code, e.what());
    return e.code == CLA_ERR_CUDA ? 3 : 2;
  }
}
