// placeholder, replaced below
#include "cla_common.cuh"
namespace cla {
int64_t fast_plan_build(Matrix*) { return CLA_OK; }
void fast_plan_free(Matrix*) {}
int64_t fast_rmm_vec(Matrix*, const double*, double*, cudaStream_t) { return 0; }
int64_t fast_lmm_vec(Matrix*, const double*, double*, cudaStream_t) { return 0; }
}
