// Host-side ternary packing (the reference's PackedTensor::pack / unpack) and the
// device kernel that converts the reference's packed bytes into the tiled streaming
// layout described in bt_common.cuh.
#include <math.h>
#include <string.h>

#include "bt_common.cuh"

namespace bt {

// Re-encode one byte of four reference codes (00/01/10/11 = 0/+1/-1/0,
// kernels/packing.rs:9-13, kernels/cpu.rs:59) into four fields u = t + 1.
__device__ __forceinline__ uint32_t recode_byte(uint32_t byte) {
    uint32_t out = 0;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        uint32_t c = (byte >> (2 * r)) & 3u;
        uint32_t u = (c == 1u) ? 2u : ((c == 2u) ? 0u : 1u);
        out |= u << (2 * r);
    }
    return out;
}

__global__ void retile_kernel(const uint8_t* __restrict__ src, int64_t n_out, int64_t kq,
                              int n_bases, uint8_t* __restrict__ tiles, int64_t row_tiles,
                              int64_t k_tiles) {
    const int64_t per_basis = row_tiles * k_tiles * kTileBytes;
    const int64_t total = per_basis * n_bases;
    for (int64_t ob = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; ob < total;
         ob += (int64_t)gridDim.x * blockDim.x) {
        const int b = (int)(ob / per_basis);
        const int64_t in_basis = ob % per_basis;
        const int64_t tile = in_basis / kTileBytes;
        const int within = (int)(in_basis % kTileBytes);
        const int64_t rt = tile / k_tiles, kt = tile % k_tiles;
        const int half = within >> 9;
        const int lane = (within & 511) >> 4;
        const int byte = within & 15;
        const int g = lane >> 2, t = lane & 3;
        const int64_t row = rt * kTileRows + half * 8 + g;
        const int64_t col = kt * (kTileK / 4) + t * 16 + byte;  // in bytes = 4 inputs
        uint32_t v = 0x55u;                                      // four zero weights
        if (row < n_out && col < kq) v = recode_byte(src[(row * kq + col) * n_bases + b]);
        tiles[ob] = (uint8_t)v;
    }
}

cudaError_t launch_retile(const uint8_t* src_dev, int64_t n_out, int64_t k_in, int n_bases,
                          uint8_t* tiles_dev, int64_t row_tiles, int64_t k_tiles,
                          cudaStream_t stream) {
    const int64_t total = row_tiles * k_tiles * kTileBytes * n_bases;
    int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (blocks < 1) blocks = 1;
    retile_kernel<<<blocks, 256, 0, stream>>>(src_dev, n_out, k_in / 4, n_bases, tiles_dev,
                                              row_tiles, k_tiles);
    return cudaGetLastError();
}

}  // namespace bt

// ---------------------------------------------------------------------------------------
// C ABI: host packing
// ---------------------------------------------------------------------------------------
extern "C" bt_status bt_pack_ternary(const float* w, int64_t n_elem, uint8_t* out,
                                     float* scale_out) {
    if (!w || !out || !scale_out || n_elem <= 0)
        return bt::set_error(BT_ERR_ARG, "bt_pack_ternary: null pointer or empty tensor");
    // scale = mean(|w|) + 1e-6 (kernels/packing.rs:56-57); double accumulation, one
    // rounding to f32.
    double acc = 0.0;
    for (int64_t i = 0; i < n_elem; ++i) acc += fabs((double)w[i]);
    const float scale = (float)(acc / (double)n_elem) + 1e-6f;
    memset(out, 0, (size_t)((n_elem + 3) / 4));
    for (int64_t i = 0; i < n_elem; ++i) {
        float q = roundf(w[i] / scale);  // round, then clamp (packing.rs:61-65)
        q = q > 1.0f ? 1.0f : (q < -1.0f ? -1.0f : q);
        const unsigned code = q > 0.5f ? 1u : (q < -0.5f ? 2u : 0u);
        out[i >> 2] |= (uint8_t)(code << ((i & 3) * 2));
    }
    *scale_out = scale;
    return BT_OK;
}

extern "C" bt_status bt_unpack_ternary(const uint8_t* packed, int64_t n_elem, float scale,
                                       float* out) {
    if (!packed || !out || n_elem < 0)
        return bt::set_error(BT_ERR_ARG, "bt_unpack_ternary: null pointer");
    for (int64_t i = 0; i < n_elem; ++i) {
        const unsigned code = (packed[i >> 2] >> ((i & 3) * 2)) & 3u;
        out[i] = (code == 1u ? 1.0f : (code == 2u ? -1.0f : 0.0f)) * scale;
    }
    return BT_OK;
}

// Legacy one-byte-per-weight layout [n_out, k_in/4, n_bases, 4] (int8 values -1 / 0 / +1 stored as
// bytes 255 / 0 / 1; pack_interleaved_blocks, tools/conversion/convert_adaptive.py:43-83, read by
// adaptive_gemm_n3_kernel_f32, kernels/adaptive_bit_op.cu:74-161) -> the 2-bit checkpoint layout
// [n_out, k_in/4, n_bases] that bt_linear_create takes.  Any other byte value is an error.
extern "C" bt_status bt_convert_l3_to_l2(const int8_t* l3_host, int64_t n_out, int64_t k_in, int n_bases,
                                         uint8_t* l2_out_host) {
    if (!l3_host || !l2_out_host) return bt::set_error(BT_ERR_ARG, "bt_convert_l3_to_l2: null pointer");
    if (n_out <= 0 || k_in <= 0 || n_bases < 1 || n_bases > 8)
        return bt::set_error(BT_ERR_SHAPE, "bt_convert_l3_to_l2: bad shape [%lld, %lld] x %d bases", (long long)n_out,
                             (long long)k_in, n_bases);
    if (k_in % 4 != 0) return bt::set_error(BT_ERR_ALIGN, "bt_convert_l3_to_l2: in_features %lld is not a multiple of 4", (long long)k_in);
    const int64_t blocks = n_out * (k_in / 4);
    for (int64_t blk = 0; blk < blocks; ++blk) {
        for (int b = 0; b < n_bases; ++b) {
            const int8_t* src = l3_host + (blk * n_bases + b) * 4;
            unsigned byte = 0;
            for (int r = 0; r < 4; ++r) {
                const int v = src[r];
                if (v < -1 || v > 1)
                    return bt::set_error(BT_ERR_ARG, "bt_convert_l3_to_l2: weight value %d at block %lld is not ternary", v, (long long)blk);
                byte |= (v > 0 ? 1u : (v < 0 ? 2u : 0u)) << (2 * r);
            }
            l2_out_host[blk * n_bases + b] = (uint8_t)byte;
        }
    }
    return BT_OK;
}
