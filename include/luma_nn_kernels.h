/*
 * Kernels of luma's math-path attention that sit next to the flash-attention path, as a C ABI.
 *
 * luma_softmax_<T>: softmax over the last dimension of a dense row-major (num_rows, row_size)
 * matrix, f32 / f16 / bf16 storage, arithmetic in f32, output rounded to nearest even.
 * Replaces the kernels softmax_f32 / softmax_f16 / softmax_bf16 of luma-cuda/kernels/nn.cu:21-76
 * (same arguments: num_rows, row_size, input, output), which luma-cuda launches from
 * luma-cuda/src/ops/nn_provide.rs:10-70 (launch_softmax) for Tensor::softmax on the last dimension — the softmax of
 * luma-tensor/src/ops/nn/attention.rs:36 on the CUDA math path. The reference loads those kernels
 * as PTX by name; a maintainer binds these symbols in that launch wrapper instead.
 * In-place operation (output == input) is allowed. A row that holds only -inf gives NaN, as the
 * reference's arithmetic does. Status codes and flash_attn_last_error() as in flash_attn.h.
 */
#ifndef LUMA_B200_LUMA_NN_KERNELS_H_
#define LUMA_B200_LUMA_NN_KERNELS_H_

#include "flash_attn.h"

#ifdef __cplusplus
extern "C" {
#endif

int luma_softmax_f32(const float* input, float* output, long long num_rows, int row_size, void* stream);
int luma_softmax_f16(const flash_attn_f16_t* input, flash_attn_f16_t* output, long long num_rows, int row_size,
                     void* stream);
int luma_softmax_bf16(const flash_attn_bf16_t* input, flash_attn_bf16_t* output, long long num_rows, int row_size,
                      void* stream);

#ifdef __cplusplus
}
#endif

#endif
