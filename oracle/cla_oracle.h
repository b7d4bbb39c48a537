/*
 * CPU oracle for the SystemDS compressed-linear-algebra (CLA) matrix-multiply path.
 *
 * TEST INFRASTRUCTURE ONLY. This library is a host-side restatement of the reference's
 * Java algorithms (file:line citations are given beside every function in cla_oracle.cpp).
 * It is the checker for the CUDA path and the timed CPU baseline; it is never linked into,
 * imported by, or called from the product library.
 *
 * Parity status: the index-structure formats (OLE/RLE bitmaps, byte/char offsets, map types)
 * are pinned by the exact arrays of the reference's own unit tests (tests/golden). The products
 * are pinned by the reference's closed-form pre-aggregation tests and by agreement with a
 * long-double dense evaluation, which is the reference's own test oracle (compressed result vs
 * uncompressed operator). OLE products: parity unpinned (the reference has no arithmetic for OLE).
 */
#ifndef CLA_ORACLE_H
#define CLA_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* map types, in the order of MapToFactory.MAP_TYPE */
enum { OCL_MAP_ZERO = 0, OCL_MAP_BIT = 1, OCL_MAP_UBYTE = 2, OCL_MAP_BYTE = 3, OCL_MAP_CHAR = 4,
       OCL_MAP_CHAR_BYTE = 5, OCL_MAP_INT = 6 };
/* offset types */
enum { OCL_OFF_EMPTY = 0, OCL_OFF_SINGLE = 1, OCL_OFF_TWO = 2, OCL_OFF_BYTE = 3, OCL_OFF_CHAR = 4 };
/* mmchain types (MapMultChain.ChainType) */
enum { OCL_CHAIN_XtXv = 0, OCL_CHAIN_XtwXv = 1 };

/* ---- format level -------------------------------------------------------------------------- */
int ocl_map_type_for(int64_t size, int64_t unique);
/* returns the encoded length (uint16 units); writes at most cap entries; -1 if input empty */
int64_t ocl_ole_gen_offset_bitmap(const int32_t* offsets, int64_t len, uint16_t* out, int64_t cap);
int64_t ocl_rle_gen_bitmap(const int32_t* offsets, int64_t len, uint16_t* out, int64_t cap);
/* OffsetFactory.createOffset: picks the type, encodes. out must hold 2*cap bytes when the result
 * is char. Returns the encoded length in elements (bytes or chars); flags bit0 = noZero, bit1 = noOverHalf */
int64_t ocl_offset_create(const int32_t* idx, int64_t n, int32_t* type, int32_t* first, int32_t* last,
                          void* out, int64_t cap, int32_t* flags);
/* walks the iterator (first, then next() until last) and returns the number of rows written */
int64_t ocl_offset_decode(int32_t type, int32_t first, int32_t last, const void* data, int64_t len,
                          int32_t* rows, int64_t cap);
/* decode a map into int32 ids */
void ocl_map_decode(int32_t type, const void* data, const void* data2, int64_t size, int32_t* ids);

/* ---- matrix level -------------------------------------------------------------------------- */
typedef struct ocl_matrix ocl_matrix;
ocl_matrix* ocl_create(int32_t nRows, int32_t nCols);
void ocl_destroy(ocl_matrix*);
int ocl_add_ddc(ocl_matrix*, const int32_t* cols, int32_t gCols, const double* dict, int32_t nVals,
                int32_t mapType, const void* map, const void* map2, int64_t mapSize);
/* SDC family: defaultTuple == NULL -> *Zeros; map == NULL (mapType ZERO) -> *Single* */
int ocl_add_sdc(ocl_matrix*, const int32_t* cols, int32_t gCols, const double* dict, int32_t nVals,
                const double* defaultTuple, int32_t offType, int32_t first, int32_t last,
                const void* offData, int64_t offLen, int32_t mapType, const void* map, const void* map2,
                int64_t mapSize);
int ocl_add_rle(ocl_matrix*, const int32_t* cols, int32_t gCols, const double* dict, int32_t nVals,
                const int32_t* ptr, const uint16_t* data, int64_t dataLen);
int ocl_add_ole(ocl_matrix*, const int32_t* cols, int32_t gCols, const double* dict, int32_t nVals,
                const int32_t* ptr, const uint16_t* data, int64_t dataLen);
int ocl_add_uncompressed(ocl_matrix*, const int32_t* cols, int32_t gCols, const double* values);
int ocl_add_const(ocl_matrix*, const int32_t* cols, int32_t gCols, const double* tuple);
int ocl_add_empty(ocl_matrix*, const int32_t* cols, int32_t gCols);

int32_t ocl_num_groups(const ocl_matrix*);
int64_t ocl_compressed_bytes(const ocl_matrix*);
/* per-row tuple id of group g (-1 where the row holds the default / zero tuple; row index for UNC) */
void ocl_group_row_ids(const ocl_matrix*, int32_t g, int32_t* ids);
/* AColGroupValue.getCounts for group g (nVals entries) */
void ocl_group_counts(const ocl_matrix*, int32_t g, int64_t* counts);

/* products; k = thread budget (as the instruction's k); all dense row-major FP64 */
void ocl_decompress(const ocl_matrix*, double* out, int k);
void ocl_rmm(const ocl_matrix*, const double* V, int32_t vCols, double* out, int k);
void ocl_lmm(const ocl_matrix*, const double* Yt, int32_t yRows, double* out, int k);
void ocl_tsmm(const ocl_matrix*, double* out, int k, int allowFallback);
void ocl_mmchain(const ocl_matrix*, const double* v, const double* w, int ctype, double* out, int k);
/* t(left) %*% right on two compressed blocks with the same number of rows; out [left.nCols x right.nCols] */
void ocl_tmm(const ocl_matrix* left, const ocl_matrix* right, double* out, int k);

/* dense long-double evaluation of the same products from the decompressed matrix */
void ocl_dense_rmm_ld(const double* X, int64_t n, int32_t m, const double* V, int32_t vCols, double* out);
void ocl_dense_lmm_ld(const double* X, int64_t n, int32_t m, const double* Yt, int32_t yRows, double* out);
void ocl_dense_tsmm_ld(const double* X, int64_t n, int32_t m, double* out);

int ocl_max_threads(void);
#ifdef __cplusplus
}
#endif
#endif
