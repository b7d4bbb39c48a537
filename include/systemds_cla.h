/*
 * systemds_cla.h -- C ABI of the B200 compressed-linear-algebra (CLA) matrix-multiply library.
 *
 * The library owns device-resident copies of the column groups of a SystemDS
 * CompressedMatrixBlock and runs the compressed matrix products on the GPU. Every entry point
 * is plain C (pointers and sizes only); the JNI shim in systemds_b200/csrc/cla_jni.cpp maps
 * 1:1 onto these calls. File:line citations name the reference interface each call replaces,
 * by path below src/main/java/org/apache/sysds/ of the reference project.
 *
 * Conventions (those of the reference's native BLAS bridge, utils/NativeHelper.java:361-418 and
 * src/main/cpp/systemds.cpp:59-82): dense operands are row-major FP64; product calls return the
 * number of non-zeros of the result (>= 0) so the caller can setNonZeros(), or a negative
 * CLA_ERR_* code. There is no CPU fallback: without a usable CUDA device every call fails.
 *
 * Host buffers may be ordinary (pageable) memory, as the arrays a JVM hands over are: transfers of
 * 4 MB and more from or to memory that is neither pinned nor registered go through a ring of pinned
 * slices owned by the handle (32 MB, allocated at the first such call), moved by a few host threads
 * of the calling process for the duration of the call (environment: CLA_STAGE_THREADS, 0 = plain
 * cudaMemcpyAsync). Pinned and registered buffers are copied asynchronously as they are.
 *
 * Threading: calls on one handle are serialised by an internal mutex; different handles may be
 * used concurrently. The thread budget "k" of the reference's calls has no meaning here.
 * Device-buffer calls (cla_*_dev) return once their work is enqueued on the caller's stream; all
 * calls on a handle share that handle's scratch buffers, so the library orders them on the device
 * as well: a call that arrives on another stream than the handle's previous call waits (event
 * wait on the device, not on the host) until that call's kernels have finished. A kernel's
 * self-check that trips in a device-buffer call is reported by the next cla_stats_get or
 * host-buffer call on the handle (CLA_ERR_DEVICE_CHECK); callers that never make one should poll
 * cla_stats_get. The right products (X %*% v, X %*% V), the specialised left vector product and
 * the chain built from them form every output cell's sum in a fixed order and are reproducible
 * bit for bit; the general left product, the self-product and the constant-column terms combine
 * partial sums with floating-point atomics and are reproducible to rounding only.
 */
#ifndef SYSTEMDS_CLA_H
#define SYSTEMDS_CLA_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define CLA_OK 0
#define CLA_ERR_BAD_HANDLE (-1)
#define CLA_ERR_BAD_ARG (-2)
#define CLA_ERR_UNSUPPORTED (-3)
#define CLA_ERR_SHAPE (-4)
#define CLA_ERR_CUDA (-5)
#define CLA_ERR_STATE (-6)   /* call order violated (e.g. product before finalize) */
#define CLA_ERR_NOMEM (-7)
#define CLA_ERR_DEVICE_CHECK (-8) /* a kernel's self-check tripped (index out of range in an index structure) */

/* AMapToData storage classes, in the order of MapToFactory.MAP_TYPE
 * (runtime/compress/colgroup/mapping/MapToFactory.java:38-40). Arrays are passed in the JVM's
 * in-memory form: BIT = long[] LSB-first (MapToBit.java:100-103), UBYTE/BYTE = byte[],
 * CHAR = char[] (u16), CHAR_BYTE = char[] + byte[] (id = c + (b << 16)), INT = int[]. */
#define CLA_MAP_ZERO 0
#define CLA_MAP_BIT 1
#define CLA_MAP_UBYTE 2
#define CLA_MAP_BYTE 3
#define CLA_MAP_CHAR 4
#define CLA_MAP_CHAR_BYTE 5
#define CLA_MAP_INT 6

/* AOffset storage classes (runtime/compress/colgroup/offset/OffsetFactory.java:105-149).
 * BYTE covers OffsetByte, OffsetByteNZ and OffsetByteUNZ (same byte stream; the NZ variants
 * simply contain no zero byte); CHAR covers OffsetChar. */
#define CLA_OFF_EMPTY 0
#define CLA_OFF_SINGLE 1
#define CLA_OFF_TWO 2
#define CLA_OFF_BYTE 3
#define CLA_OFF_CHAR 4

/* MapMultChain.ChainType (lops/MapMultChain.java) */
#define CLA_CHAIN_XtXv 0
#define CLA_CHAIN_XtwXv 1

typedef int64_t cla_handle;

/* Per-handle counters, the device-side analogue of utils/DMLCompressionStatistics.java:24-125. */
typedef struct cla_stats {
  int64_t n_rows, n_cols, n_groups;
  int64_t device_bytes;      /* bytes held on the device for this matrix */
  int64_t index_bytes;       /* bytes of index structures + dictionaries (one pass reads these) */
  int64_t calls_rmm, calls_lmm, calls_tsmm, calls_mmchain, calls_decompress;
  int64_t kernel_launches;   /* launches issued by this handle since creation */
  double last_kernel_ms;     /* device time of the last host-buffer product call (CUDA events) */
  double main_kernel_ms;     /* with profiling on: summed device time of the dominant kernel of each product call */
  int64_t main_kernel_count; /* ... and how many launches that sum covers */
} cla_stats;

/* ---- life cycle ---------------------------------------------------------------------------
 * Replaces the construction of a CompressedMatrixBlock's group list
 * (runtime/compress/CompressedMatrixBlock.java:108-132). */
cla_handle cla_create(int32_t nRows, int32_t nCols, int32_t overlapping);
int64_t cla_destroy(cla_handle h);
/* Uploads all groups to CUDA device `device`, builds skip indexes and launch plans.
 * After this call the host arrays given to cla_add_group_* are no longer referenced. */
int64_t cla_finalize(cla_handle h, int32_t device);
/* Copies the message of the calling thread's last failed call into buf; returns its length. */
int64_t cla_last_error(char* buf, int64_t cap);
/* Also reports (as CLA_ERR_DEVICE_CHECK) a self-check that tripped in a kernel of an earlier device-buffer call:
 * those calls return before their kernels ran. Synchronises the handle's profiling events. */
int64_t cla_stats_get(cla_handle h, cla_stats* out);
/* Profiling switch (the analogue of the reference's -stats timers, utils/Statistics.java): when on, every
 * product call brackets its dominant kernel with CUDA events on the launching stream; cla_stats_get
 * synchronises those events and adds them to main_kernel_ms / main_kernel_count. */
int64_t cla_set_profile(cla_handle h, int32_t on);
/* Diagnostics: sustained TFLOP/s of back-to-back FP64 tensor-core instructions (DMMA m8n8k4) and of FP64 FMA on
 * `device`, the denominators of the tensor-pipe and FMA fractions reported for the kernels. About 0.1 s. */
int64_t cla_measure_fp64_peaks(int32_t device, double* dmmaTflops, double* dfmaTflops);

/* Builds a handle from the serialized form of a block: replaces CompressedMatrixBlock.read(DataInput)
 * (runtime/compress/CompressedMatrixBlock.java:486-496) and ColGroupIO.readGroups (colgroup/ColGroupIO.java:48-63).
 * `bytes` is the big-endian stream CompressedMatrixBlock.write(DataOutput) produced (what a Spark broadcast, an
 * evicted buffer-pool entry or a binary file holds). Returns the new, not yet finalized handle (> 0) or a CLA_ERR_*
 * code: CLA_ERR_BAD_ARG for a truncated stream, CLA_ERR_UNSUPPORTED for classes outside this library (LZW / delta /
 * linear-functional groups, quantised / delta / placeholder / identity-slice dictionaries, de-duplicated dense
 * blocks). *nonZeros receives the header's count, *consumed the bytes read; both may be NULL. */
cla_handle cla_read_block(const uint8_t* bytes, int64_t len, int64_t* nonZeros, int64_t* consumed);

/* ---- group registration (host arrays are copied) -------------------------------------------
 * Each returns the index of the new group (>= 0) or a CLA_ERR_* code.
 * colIdx: the group's IColIndex flattened to int32 (colgroup/indexes/ColIndexFactory.java:38-118).
 * dict:   Dictionary values, row-major [nVals x gCols] (colgroup/dictionary/Dictionary.java:94-97). */

/* ColGroupDDC {_colIndexes, _dict, _data} (colgroup/ColGroupDDC.java:79-89) */
int64_t cla_add_group_ddc(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dict, int32_t nVals,
                          int32_t mapType, const void* map, const void* mapHi, int64_t mapSize);
/* ColGroupSDC / SDCZeros / SDCSingle / SDCSingleZeros (colgroup/ColGroupSDC.java:67-99,
 * ColGroupSDCZeros.java:75-92, ColGroupSDCSingle.java:83-105, ColGroupSDCSingleZeros.java:82-93).
 * defaultTuple NULL = the *Zeros variants; map NULL = the *Single* variants (one tuple, no map).
 * offData holds offLen u8 (BYTE) or u16 (CHAR) deltas; nOffsets = AOffset.getSize(). */
int64_t cla_add_group_sdc(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dict, int32_t nVals,
                          const double* defaultTuple, int32_t offType, int32_t offsetToFirst, int32_t offsetToLast,
                          const void* offData, int64_t offLen, int64_t nOffsets, int32_t mapType, const void* map,
                          const void* mapHi);
/* ColGroupRLE {_ptr, _data} (colgroup/AColGroupOffset.java:39-55, ColGroupRLE.java:114-117) */
int64_t cla_add_group_rle(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dict, int32_t nVals,
                          const int32_t* ptr, const uint16_t* data, int64_t dataLen);
/* ColGroupOLE {_ptr, _data} (colgroup/ColGroupOLE.java:558-599). The reference has no arithmetic for
 * this group (its product methods throw); here it takes part in every product. */
int64_t cla_add_group_ole(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dict, int32_t nVals,
                          const int32_t* ptr, const uint16_t* data, int64_t dataLen);
/* ColGroupUncompressed {_data} dense [nRows x gCols] (colgroup/ColGroupUncompressed.java:84) */
int64_t cla_add_group_uncompressed(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* values);
/* The same two groups when the index map / dense block already lives in device memory (same layouts; colIdx and
 * dict stay host arrays). The device buffer is read by cla_finalize (device-to-device copy, ids checked by a
 * kernel: an id at or above nVals makes cla_finalize fail with CLA_ERR_BAD_ARG) and must stay valid and unchanged
 * until cla_finalize has returned. Maps: MapToBit, MapToUByte, MapToByte, MapToChar or MapToInt. These have no
 * counterpart in the reference, whose column groups always live on the JVM heap (colgroup/ColGroupDDC.java:79-89). */
int64_t cla_add_group_ddc_dev(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dict, int32_t nVals,
                              int32_t mapType, const void* dMap, int64_t mapSize);
int64_t cla_add_group_uncompressed_dev(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* dValues);
/* ColGroupConst (one tuple) and ColGroupEmpty; both fold into the constant row vector that
 * lib/CLALibUtils.java:188-206 (filterGroups) builds. */
int64_t cla_add_group_const(cla_handle h, const int32_t* colIdx, int32_t gCols, const double* tuple);
int64_t cla_add_group_empty(cla_handle h, const int32_t* colIdx, int32_t gCols);

/* ---- products, host buffers (copies to and from the device happen inside the call) ----------
 * cla_rmm      replaces lib/CLALibRightMultBy.java:57  rightMultByMatrix(m1, m2, ret, k): out[nRows x vCols] = X * V
 * cla_lmm      replaces lib/CLALibLeftMultBy.java:126  leftMultByMatrix(right, left, ret, k):
 *              out[yRows x nCols] = Yt * X with Yt [yRows x nRows] (the already transposed left operand)
 * cla_tsmm     replaces lib/CLALibTSMM.java:59  leftMultByTransposeSelf(cmb, ret, k): out[nCols x nCols] = t(X) X
 * cla_mmchain  replaces lib/CLALibMMChain.java:92  mmChain(x, v, w, out, ctype, k): out[nCols] = t(X) (w * (X v))
 * cla_decompress replaces lib/CLALibDecompress.java:56  decompress(cmb, k): out[nRows x nCols] */
int64_t cla_rmm(cla_handle h, const double* V, int32_t vRows, int32_t vCols, double* out);
/* X * V kept compressed: replaces lib/CLALibRightMultBy.java:51 rightMultByMatrix(m1, m2, ret, k, allowOverlap = true),
 * i.e. RMMOverlapping (:157-201). Returns the handle (> 0, finalized, same device) of an overlapping block
 * [nRows x vCols] whose groups share the index structures of h and hold the dictionaries D_g * V[cols_g, :]; cost is
 * proportional to the dictionaries, not to the rows (uncompressed groups excepted: their product is materialised).
 * The new block takes every call a registered block takes (products, decompress, aggregates; t(h) %*% result through
 * cla_tmm is the reference's overlapping-intermediate form of the matrix-multiply chain, lib/CLALibMMChain.java:109-122).
 * It may outlive h: destroying h first only retires the handle, its device memory is released with the last such
 * result. The _dev form takes V in device memory and enqueues on `stream` (it still synchronises that stream). */
cla_handle cla_rmm_overlapping(cla_handle h, const double* V, int32_t vRows, int32_t vCols);
cla_handle cla_rmm_overlapping_dev(cla_handle h, const double* dV, int32_t vRows, int32_t vCols, void* stream);
int64_t cla_lmm(cla_handle h, const double* Yt, int32_t yRows, double* out);
int64_t cla_tsmm(cla_handle h, double* out);
int64_t cla_mmchain(cla_handle h, const double* v, const double* w, int32_t ctype, double* out);
int64_t cla_decompress(cla_handle h, double* out);

/* t(left) %*% right on two compressed blocks with the same number of rows, finalized on the same device:
 * replaces lib/CLALibLeftMultBy.java:100  leftMultByMatrixTransposed(right, left, ret, k) with a compressed
 * left operand (the compressed x compressed case of lib/CLALibMatrixMult.java:96-124).
 * out [left.nCols x right.nCols], dense row-major. left == right is allowed (same result as cla_tsmm). */
int64_t cla_tmm(cla_handle left, cla_handle right, double* out);

/* Sum aggregates on the compressed block, the uak+ / uark+ / uack+ cases of lib/CLALibCompAgg.java
 * (colgroup/AColGroupCompressed.java:140-205 computeSum / computeRowSums / computeColSums):
 * CLA_AGG_COL_* -> out[nCols], CLA_AGG_ROW_* -> out[nRows], CLA_AGG_SUM / MIN / MAX -> out[1]. Host buffer. */
#define CLA_AGG_COL_SUMS 0
#define CLA_AGG_ROW_SUMS 1
#define CLA_AGG_SUM 2
/* min / max (uacmin, uacmax, uarmin, uarmax, uamin, uamax). Column-wise and full extrema of a block whose groups
 * do not overlap follow the reference's dictionary-based definition (AColGroupCompressed.computeMxx /
 * computeColMxx: every dictionary entry counts, plus the default tuple or 0 where rows fall outside the
 * index structure); row-wise extrema and overlapping blocks go through decompressed row chunks. */
#define CLA_AGG_COL_MINS 3
#define CLA_AGG_COL_MAXS 4
#define CLA_AGG_ROW_MINS 5
#define CLA_AGG_ROW_MAXS 6
#define CLA_AGG_MIN 7
#define CLA_AGG_MAX 8
int64_t cla_unary_agg(cla_handle h, int32_t op, double* out);

/* ---- products, device buffers --------------------------------------------------------------
 * Same semantics; every pointer is a device address on the handle's device, `stream` is a
 * cudaStream_t (NULL = the legacy default stream). The call enqueues work and returns CLA_OK
 * without synchronising; no non-zero count is produced. Used for row-sharded multi-GPU runs,
 * where the caller all-reduces the partial results of cla_lmm_dev / cla_tsmm_dev / cla_mmchain_dev. */
int64_t cla_rmm_dev(cla_handle h, const double* dV, int32_t vRows, int32_t vCols, double* dOut, void* stream);
int64_t cla_lmm_dev(cla_handle h, const double* dYt, int32_t yRows, double* dOut, void* stream);
int64_t cla_tsmm_dev(cla_handle h, double* dOut, void* stream);
int64_t cla_tmm_dev(cla_handle left, cla_handle right, double* dOut, void* stream);
/* decompress into a device buffer of nRows x nCols doubles (lib/CLALibDecompress.java:56) */
int64_t cla_decompress_dev(cla_handle h, double* dOut, void* stream);
/* dU: caller-provided scratch of nRows doubles for u = X v (may be NULL: the handle then keeps its own) */
int64_t cla_mmchain_dev(cla_handle h, const double* dV, const double* dW, int32_t ctype, double* dOut, double* dU,
                        void* stream);
/* Row sharding needs no special entry point: a handle that holds rows [a, b) of a taller matrix
 * yields the exact product of those rows (constant columns included), so the partial results of
 * cla_lmm_dev / cla_tsmm_dev / cla_tmm_dev / cla_mmchain_dev over all shards simply add up. */

/* t(y) %*% X (one left row) that performs no device allocation. It has no counterpart in the reference.
 * For hosts that must not allocate when they call in -- a runtime whose own pool owns all device memory, or a loop
 * that cannot afford the device-wide synchronisation inside cudaMalloc -- the kernel's scratch (per-CTA partial
 * sums, the row sum of dY) is a fixed array inside the library, about 450 KB, held by every GPU that loads the
 * library until the process exits. Inputs and output are still the caller's: dY [nRows] and dOut [nCols] are
 * device addresses, dY 16-byte aligned. Same result as cla_lmm_dev with yRows = 1.
 * Limits: the matrix must consist of dense-map (DDC) groups with at most 256 tuples and 1-byte (or 1-bit) maps,
 * and need at most 512 partial-sum rows (one per launched CTA: the SM count, or the number of 112-column chunks if
 * that is larger); otherwise CLA_ERR_UNSUPPORTED is returned and nothing runs.
 * The first call on a device looks up the array's device address; make that call outside any stream capture.
 * All calls share the array and it keeps the previous call's contents (what must start at zero is cleared on the
 * stream first), so two calls whose kernels overlap on the GPU -- different streams or handles -- race. */
int64_t cla_lmm_vec_noalloc_dev(cla_handle h, const double* dY, double* dOut, void* stream);

/* ---- The sum over the ranks that ends a product on a row-sharded block (one process per GPU, one node) ----
 * It has no counterpart in the reference, whose compressed products run in one JVM. Each rank holds the rows of its
 * shard; t(y) %*% X, t(X) %*% X and the chain give per-rank partial results that add up. cla_allreduce_dev sums n
 * doubles in place over all ranks with one kernel per rank over NVLink peer memory (stores into every peer's
 * buffer, a flag, a bounded wait, the sum in rank order: all ranks end with identical bits). Setup: every rank
 * calls cla_comm_create, the host passes the 64-byte handles of all ranks (rank order) to cla_comm_connect.
 * All ranks must call cla_allreduce_dev the same number of times in the same order. A rank that does not arrive
 * within the time limit (default 2 s) makes the others fill their result with NaN; cla_comm_status (which
 * synchronises the device) then returns CLA_ERR_DEVICE_CHECK naming the missing rank, and the comm stays usable.
 * cla_comm_connect(comm, NULL) maps every rank to the caller's own buffer (single-process checks). */
#define CLA_COMM_HANDLE_BYTES 64
int64_t cla_comm_create(int32_t device, int32_t rank, int32_t world, int64_t maxDoubles, void* ipcHandleOut);
int64_t cla_comm_connect(int64_t comm, const void* allHandles);
int64_t cla_comm_set_timeout_ms(int64_t comm, int64_t ms);
int64_t cla_allreduce_dev(int64_t comm, double* dBuf, int64_t n, void* stream);
int64_t cla_comm_status(int64_t comm);
int64_t cla_comm_destroy(int64_t comm);

/* ---- decoded index structures (for bit-exact checks and for f2-style consumers) -------------
 * ids[nRows]: dictionary id of every row of group g, -1 where the row holds the default (or zero)
 * tuple; for an uncompressed group the row number. Computed by the device decode kernels.
 * counts[nVals]: AColGroupValue.getCounts (colgroup/AColGroupValue.java:94-96). */
int64_t cla_group_decode(cla_handle h, int32_t g, int32_t* ids);
int64_t cla_group_counts(cla_handle h, int32_t g, int64_t* counts);

#ifdef __cplusplus
}
#endif
#endif
