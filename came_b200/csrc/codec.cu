// Stand-alone blockwise codec kernels (not on the step's hot path, where the codec is fused into the
// step kernels).  Bit-exact with came_pytorch/blockwise_quantization.py:66-124: IEEE division,
// round-half-even, zero padding of the last block.
#include "common.cuh"
#include "launch.h"

namespace came {

template <bool SIGNED>
__global__ void __launch_bounds__(QBLOCK) k_quant_flat(const float* __restrict__ src, void* __restrict__ q,
                                                       float* __restrict__ absmax, int64_t n) {
    __shared__ float red[33];
    const int64_t idx = (int64_t)blockIdx.x * QBLOCK + threadIdx.x;
    const bool valid = idx < n;
    const float x = valid ? src[idx] : 0.0f;
    // signed: max |x|; unsigned: max x over the zero-padded block (blockwise_quantization.py:73-79)
    const float a = fix_absmax(block_max(SIGNED ? fabsf(x) : x, red));
    if (threadIdx.x == 0) absmax[blockIdx.x] = a;
    if (valid) {
        if (SIGNED) reinterpret_cast<int8_t*>(q)[idx] = (int8_t)quant_i8_div(x, a);
        else reinterpret_cast<uint8_t*>(q)[idx] = (uint8_t)quant_u8_div(x, a);
    }
}

template <bool SIGNED>
__global__ void __launch_bounds__(QBLOCK) k_dequant_flat(const void* __restrict__ q, const float* __restrict__ absmax,
                                                         float* __restrict__ dst, int64_t n) {
    const int64_t idx = (int64_t)blockIdx.x * QBLOCK + threadIdx.x;
    if (idx >= n) return;
    const float a = absmax[blockIdx.x];
    if (SIGNED) dst[idx] = (float)reinterpret_cast<const int8_t*>(q)[idx] * (a / QMAX_I8);
    else dst[idx] = (float)reinterpret_cast<const uint8_t*>(q)[idx] * (a / QMAX_U8);
}

// one CTA of 256 threads per 16x16 tile
__global__ void __launch_bounds__(QBLOCK) k_quant_tile(const float* __restrict__ src, int8_t* __restrict__ q,
                                                       float* __restrict__ absmax, int rows, int cols, int tile_cols) {
    __shared__ float red[33];
    const int ty = blockIdx.x / tile_cols, tx = blockIdx.x - ty * tile_cols;
    const int row = ty * TILE + (threadIdx.x >> 4), col = tx * TILE + (threadIdx.x & 15);
    const bool valid = row < rows && col < cols;
    const float x = valid ? src[(int64_t)row * cols + col] : 0.0f;
    const float a = fix_absmax(block_max(fabsf(x), red));
    if (threadIdx.x == 0) absmax[blockIdx.x] = a;
    if (valid) q[(int64_t)row * cols + col] = (int8_t)quant_i8_div(x, a);
}

__global__ void __launch_bounds__(QBLOCK) k_dequant_tile(const int8_t* __restrict__ q, const float* __restrict__ absmax,
                                                         float* __restrict__ dst, int rows, int cols, int tile_cols) {
    const int ty = blockIdx.x / tile_cols, tx = blockIdx.x - ty * tile_cols;
    const int row = ty * TILE + (threadIdx.x >> 4), col = tx * TILE + (threadIdx.x & 15);
    if (row >= rows || col >= cols) return;
    const float a = absmax[blockIdx.x];
    const int64_t idx = (int64_t)row * cols + col;
    dst[idx] = a > 0.0f ? (float)q[idx] * (a / QMAX_I8) : 0.0f;
}

static inline int64_t nblocks(int64_t n) { return n <= 0 ? 1 : (n + QBLOCK - 1) / QBLOCK; }

cudaError_t launch_quantize_blockwise(const float* src, void* q, float* absmax, int64_t n, bool is_signed,
                                      cudaStream_t st) {
    const unsigned grid = (unsigned)nblocks(n);
    if (is_signed) k_quant_flat<true><<<grid, QBLOCK, 0, st>>>(src, q, absmax, n);
    else k_quant_flat<false><<<grid, QBLOCK, 0, st>>>(src, q, absmax, n);
    return cudaGetLastError();
}

cudaError_t launch_dequantize_blockwise(const void* q, const float* absmax, float* dst, int64_t n, bool is_signed,
                                        cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    const unsigned grid = (unsigned)nblocks(n);
    if (is_signed) k_dequant_flat<true><<<grid, QBLOCK, 0, st>>>(q, absmax, dst, n);
    else k_dequant_flat<false><<<grid, QBLOCK, 0, st>>>(q, absmax, dst, n);
    return cudaGetLastError();
}

cudaError_t launch_quantize_tile16(const float* src, int8_t* q, float* absmax, int64_t rows, int64_t cols,
                                   cudaStream_t st) {
    const int tr = (int)((rows + TILE - 1) / TILE), tc = (int)((cols + TILE - 1) / TILE);
    k_quant_tile<<<(unsigned)(tr * tc), QBLOCK, 0, st>>>(src, q, absmax, (int)rows, (int)cols, tc);
    return cudaGetLastError();
}

cudaError_t launch_dequantize_tile16(const int8_t* q, const float* absmax, float* dst, int64_t rows, int64_t cols,
                                     cudaStream_t st) {
    const int tr = (int)((rows + TILE - 1) / TILE), tc = (int)((cols + TILE - 1) / TILE);
    k_dequant_tile<<<(unsigned)(tr * tc), QBLOCK, 0, st>>>(q, absmax, dst, (int)rows, (int)cols, tc);
    return cudaGetLastError();
}

}  // namespace came
