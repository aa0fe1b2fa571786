// Prefill-sized BQ GEMM on the 5th-generation tensor cores (tcgen05 + TMEM). Under construction:
// this translation unit currently only provides its device error word.
#include "common.cuh"

namespace q38 {
unsigned int qgemm_umma_error(bool clear) { return read_tu_error(clear); }
}  // namespace q38
