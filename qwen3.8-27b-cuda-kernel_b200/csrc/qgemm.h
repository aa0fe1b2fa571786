// Internal interface between the GEMM dispatcher (qgemm.cu) and its kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/q38_kernels.h"

namespace q38 {

// Weight-streaming kernel for m <= 8 * mt, mt in {1, 2} (qgemm_stream.cu).
int qgemm_stream_launch(int mt, const __nv_bfloat16* a, int m, const q38_bq_weight& w, const q38_gemm_epilogue& ep,
                        const q38_gemm_workspace* ws, cudaStream_t s);
unsigned int qgemm_stream_error(bool clear);

// tcgen05 / TMEM kernel for m <= tok * mblocks, tok in {32, 64, 128, 256, 512} (qgemm_umma.cu); a_in_tmem: the
// decoded weights are handed to the MMA through tensor memory instead of shared memory (tok <= 256).
int qgemm_umma_launch(int tok, int mblocks, bool a_in_tmem, const __nv_bfloat16* a, int m, const q38_bq_weight& w,
                      const q38_gemm_epilogue& ep, const q38_gemm_workspace* ws, cudaStream_t s);

}  // namespace q38
