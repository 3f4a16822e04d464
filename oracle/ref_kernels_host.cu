/*
 * Host launchers around the reference project's own CUDA kernels.  TEST INFRASTRUCTURE, NOT
 * PRODUCT CODE.
 *
 * The two kernels are compiled from the reference's source files where they lie (the
 * Makefile passes their paths as REF_BIT_OP / REF_ADAPTIVE_BIT_OP; nothing is copied):
 *   crates/rust_engine/src/kernels/bit_op.cu:4-45            bit_linear_forward
 *   crates/rust_engine/src/kernels/adaptive_bit_op.cu:74-161 adaptive_gemm_n3_kernel_f32
 * The reference never launches either of them (its CUDA path unpacks on the host and calls a
 * dense GEMM, kernels/cuda.rs:21-47), so the launch geometry below follows the index
 * arithmetic inside the kernels (bit_op.cu:14-15: x = batch, y = output row;
 * adaptive_bit_op.cu:92-93: x = output row, y = batch; block of 256 as kernels/cuda.rs:125-133
 * plans it).  Buffers are host pointers; every call allocates, copies, launches, copies back
 * and frees.  Return value: 0 or the cudaError_t that failed.
 */
#include <cuda_runtime.h>
#include <stdint.h>

#include REF_BIT_OP
#include REF_ADAPTIVE_BIT_OP

#define TRY(e)                            \
    do {                                  \
        cudaError_t _e = (e);             \
        if (_e != cudaSuccess) { rc = (int)_e; goto done; } \
    } while (0)

extern "C" int ref_bit_linear_forward(const float* x_host, const uint8_t* w_host, float* y_host, float scale,
                                      int batch, int in_dim, int out_dim) {
    int rc = 0;
    float *x = nullptr, *y = nullptr;
    uint8_t* w = nullptr;
    const size_t xb = (size_t)batch * in_dim * sizeof(float), yb = (size_t)batch * out_dim * sizeof(float);
    const size_t wb = (size_t)out_dim * (size_t)(in_dim / 4);
    TRY(cudaMalloc(&x, xb));
    TRY(cudaMalloc(&y, yb));
    TRY(cudaMalloc(&w, wb));
    TRY(cudaMemcpy(x, x_host, xb, cudaMemcpyHostToDevice));
    TRY(cudaMemcpy(w, w_host, wb, cudaMemcpyHostToDevice));
    {
        const dim3 block(4, 64);
        const dim3 grid((unsigned)((batch + block.x - 1) / block.x), (unsigned)((out_dim + block.y - 1) / block.y));
        bit_linear_forward<<<grid, block>>>(x, w, y, scale, batch, in_dim, out_dim);
    }
    TRY(cudaGetLastError());
    TRY(cudaDeviceSynchronize());
    TRY(cudaMemcpy(y_host, y, yb, cudaMemcpyDeviceToHost));
done:
    cudaFree(x);
    cudaFree(y);
    cudaFree(w);
    return rc;
}

/* w_host: the legacy int8 layout [out, in/4, 3, 4] (tools/conversion/convert_adaptive.py:43-83),
 * values -1 / 0 / +1 as bytes; scales_host: 3 floats. */
extern "C" int ref_adaptive_gemm_n3(const float* x_host, const int8_t* w_host, const float* scales_host, float* y_host,
                                    int batch, int in_dim, int out_dim) {
    int rc = 0;
    float *x = nullptr, *y = nullptr, *s = nullptr;
    int8_t* w = nullptr;
    const size_t xb = (size_t)batch * in_dim * sizeof(float), yb = (size_t)batch * out_dim * sizeof(float);
    const size_t wb = (size_t)out_dim * (size_t)(in_dim / 4) * 12;
    TRY(cudaMalloc(&x, xb));
    TRY(cudaMalloc(&y, yb));
    TRY(cudaMalloc(&w, wb));
    TRY(cudaMalloc(&s, 3 * sizeof(float)));
    TRY(cudaMemcpy(x, x_host, xb, cudaMemcpyHostToDevice));
    TRY(cudaMemcpy(w, w_host, wb, cudaMemcpyHostToDevice));
    TRY(cudaMemcpy(s, scales_host, 3 * sizeof(float), cudaMemcpyHostToDevice));
    {
        const dim3 block(BLOCK_SIZE);
        const dim3 grid((unsigned)((out_dim + BLOCK_SIZE - 1) / BLOCK_SIZE), (unsigned)batch);
        adaptive_gemm_n3_kernel_f32<<<grid, block>>>(x, w, s, y, batch, in_dim, out_dim);
    }
    TRY(cudaGetLastError());
    TRY(cudaDeviceSynchronize());
    TRY(cudaMemcpy(y_host, y, yb, cudaMemcpyDeviceToHost));
done:
    cudaFree(x);
    cudaFree(y);
    cudaFree(w);
    cudaFree(s);
    return rc;
}
