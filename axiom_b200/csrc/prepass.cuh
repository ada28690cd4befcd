// prepass.cuh — operand-preparation launchers (see prepass.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

enum SplitMode { SPLIT_TF32X2 = 0, SPLIT_BF16X1 = 1, SPLIT_BF16X2 = 2, SPLIT_BF16X3 = 3 };

static inline int split_num_planes(int mode) { return mode == SPLIT_BF16X1 ? 1 : (mode == SPLIT_BF16X3 ? 3 : 2); }
static inline int split_elem_bytes(int mode) { return mode == SPLIT_TF32X2 ? 4 : 2; }

// in: fp32, either [rows, k] with pitch ld (in_is_k_major_outer = false) or
// [k, rows] with pitch ld (true).  chunk_k > 0 (row-major source only): k is cut into chunks held as
// separate [rows, chunk_k] blocks chunk_stride elements apart.  planes: [rows, pitch] each, k contiguous.
int split_planes(int mode, const float *in, int64_t rows, int64_t k, int64_t ld, bool in_is_k_major_outer,
                 void *const planes[3], int64_t pitch, int sm_count, cudaStream_t st, int64_t chunk_k = 0,
                 int64_t chunk_stride = 0);
// Both operands of a GEMM (same mode, same k) in one launch; arguments as for two split_planes calls.
int split_planes_pair(int mode, const float *a_in, int64_t a_rows, int64_t a_ld, bool a_transposed, void *const a_planes[3],
                      int64_t a_pitch, int64_t a_chunk_k, int64_t a_chunk_stride, const float *b_in, int64_t b_rows,
                      int64_t b_ld, bool b_transposed, void *const b_planes[3], int64_t b_pitch, int64_t k, int sm_count,
                      cudaStream_t st);
// planes [out_h*out_w, pitch] of the im2col matrix of one [C_in, H, W] sample (k = (c, ky, kx), zero padding)
int split_im2col(int mode, const float *in, int64_t C_in, int64_t H, int64_t W, int kh, int kw, int sh, int sw, int ph,
                 int pw, int64_t out_h, int64_t out_w, void *const planes[3], int64_t pitch, int sm_count, cudaStream_t st);
// The two operands of an implicit convolution in one launch: the images [batch][C_in][HW] -> channel-innermost planes
// [batch * HW][image_pitch], and the filter [C_out][C_in][taps] -> planes [C_out][w_pitch] with element
// tap * c_pad + c (zero for c >= C_in; c_pad even).
int split_conv_operands(int mode, const float *image, int64_t batch, int64_t C_in, int64_t HW, void *const image_planes[3],
                        int64_t image_pitch, const float *w, int64_t C_out, int taps, int c_pad, void *const w_planes[3],
                        int64_t w_pitch, int sm_count, cudaStream_t st);
int widen_i8_to_bf16(const int8_t *in, int64_t rows, int64_t k, void *out, int64_t pitch, int sm_count,
                     cudaStream_t st);
int repitch_i8(const int8_t *in, int64_t rows, int64_t k, int8_t *out, int64_t pitch, int sm_count,
               cudaStream_t st);
int requant_mult(float a_scale, const float *b_scales, float out_scale, int64_t n, float *mult,
                 cudaStream_t st);
int quantize_rows(const float *w, int64_t n, int64_t k, int8_t *q, float *scales, cudaStream_t st);

}  // namespace axb
