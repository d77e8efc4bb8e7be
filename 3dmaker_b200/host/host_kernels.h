// Small layout helpers used by the host classes: row padding / un-padding between the caller's dimensions
// and the padded (power of two, minimum 8) dimensions the kernels run on.  They replace fusedPadAndCastKernel,
// fusedUnpadAndCastKernel (modules/TinyMLP/TinyMLP.cu:23-62) and hg_padInputFloat / hg_unpadFloat /
// hg_padHalfToHalf (modules/TinyMLP/TinyMLPHashGrid.cu:11-29).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace nb {
// dst[r][c] = c < src_dim ? src[r][c] : 0, for r < rows, c < dst_dim
void pad_rows_half(const half* src, half* dst, int64_t rows, int src_dim, int dst_dim, cudaStream_t stream);
void pad_rows_float(const float* src, float* dst, int64_t rows, int src_dim, int dst_dim, cudaStream_t stream);
// dst[r][c] = src[r][c] for c < dst_dim (dst_dim <= src_dim)
void unpad_rows_float(const float* src, float* dst, int64_t rows, int src_dim, int dst_dim, cudaStream_t stream);
}  // namespace nb
