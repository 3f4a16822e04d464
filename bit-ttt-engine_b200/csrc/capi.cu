// extern "C" entry points for BitLinear: handles, workspaces, forward calls.
#include <stdarg.h>
#include <string.h>

#include <mutex>
#include <new>

#include "bt_common.cuh"

namespace bt {

// ---------------------------------------------------------------------------------------
// errors / per-device state
// ---------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

bt_status set_error(bt_status code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
void clear_error() { g_err[0] = 0; }

constexpr int kMaxDevices = 64;
struct DeviceState {
    std::mutex mu;
    bool init = false;
    int sm_count = 0;
    unsigned int* err_word = nullptr;
};
static DeviceState g_dev[kMaxDevices];

static DeviceState* device_state(int device) {
    if (device < 0 || device >= kMaxDevices) return nullptr;
    DeviceState* st = &g_dev[device];
    std::lock_guard<std::mutex> lock(st->mu);
    if (!st->init) {
        DeviceGuard guard(device);
        if (!guard.ok) return nullptr;
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return nullptr;
        st->sm_count = prop.multiProcessorCount;
        if (cudaMalloc(&st->err_word, sizeof(unsigned int)) != cudaSuccess) return nullptr;
        if (cudaMemset(st->err_word, 0, sizeof(unsigned int)) != cudaSuccess) return nullptr;
        st->init = true;
    }
    return st;
}

unsigned int* device_error_word(int device) {
    DeviceState* st = device_state(device);
    return st ? st->err_word : nullptr;
}

int device_sm_count(int device) {
    DeviceState* st = device_state(device);
    return st ? st->sm_count : 0;
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                        int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(in[i]);
}

}  // namespace bt

// ---------------------------------------------------------------------------------------
// handle types
// ---------------------------------------------------------------------------------------
#include "bt_handles.cuh"

using namespace bt;

extern "C" const char* bt_last_error(void) { return bt::g_err; }
extern "C" int bt_version(void) { return 100; }

extern "C" int bt_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

extern "C" bt_status bt_device_check(int device) {
    DeviceGuard guard(device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "bt_device_check: cannot select device %d", device);
    unsigned int* w = device_error_word(device);
    if (!w) return set_error(BT_ERR_DEVICE, "bt_device_check: device %d not usable", device);
    BT_CUDA_TRY(cudaDeviceSynchronize());
    unsigned int v = 0;
    BT_CUDA_TRY(cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost));
    if (v != 0) {
        BT_CUDA_TRY(cudaMemset(w, 0, sizeof(v)));
        return set_error(BT_ERR_TIMEOUT, "a bounded device-side wait ran out (kernel tag 0x%08x)", v);
    }
    return BT_OK;
}

// ---------------------------------------------------------------------------------------
// workspace
// ---------------------------------------------------------------------------------------
extern "C" bt_status bt_workspace_create(bt_workspace** out, int device, size_t bytes) {
    if (!out) return set_error(BT_ERR_ARG, "bt_workspace_create: null out pointer");
    *out = nullptr;
    if (bt_device_count() <= device || device < 0)
        return set_error(BT_ERR_DEVICE, "bt_workspace_create: no CUDA device %d", device);
    if (bytes == 0) bytes = (size_t)48 << 20;
    DeviceGuard guard(device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "cannot select device %d", device);
    bt_workspace* ws = new (std::nothrow) bt_workspace();
    if (!ws) return set_error(BT_ERR_NOMEM, "host allocation failed");
    ws->device = device;
    ws->bytes = bytes;
    cudaError_t e = cudaMalloc(&ws->base, bytes);
    if (e != cudaSuccess) {
        delete ws;
        return set_error(BT_ERR_NOMEM, "cudaMalloc of %zu workspace bytes failed: %s", bytes,
                         cudaGetErrorString(e));
    }
    *out = ws;
    return BT_OK;
}

extern "C" bt_status bt_workspace_destroy(bt_workspace* ws) {
    if (!ws) return BT_OK;
    DeviceGuard guard(ws->device);
    cudaFree(ws->base);
    delete ws;
    return BT_OK;
}

// ---------------------------------------------------------------------------------------
// BitLinear handle
// ---------------------------------------------------------------------------------------
extern "C" bt_status bt_linear_create(bt_linear** out, const uint8_t* packed_host, int64_t n_out,
                                      int64_t k_in, int n_bases, const float* scales_host,
                                      int device) {
    if (!out) return set_error(BT_ERR_ARG, "bt_linear_create: null out pointer");
    *out = nullptr;
    if (!packed_host || !scales_host) return set_error(BT_ERR_ARG, "bt_linear_create: null pointer");
    if (n_out <= 0 || k_in <= 0) return set_error(BT_ERR_SHAPE, "bt_linear_create: empty weight [%lld, %lld]", (long long)n_out, (long long)k_in);
    if (k_in % 4 != 0)
        return set_error(BT_ERR_ALIGN, "bt_linear_create: in_features %lld is not a multiple of 4", (long long)k_in);
    if (n_bases < 1 || n_bases > 8) return set_error(BT_ERR_ARG, "bt_linear_create: n_bases %d outside 1..8", n_bases);
    if (gemv_max_tokens((k_in + kTileK - 1) / kTileK) < 1)
        return set_error(BT_ERR_SHAPE, "bt_linear_create: in_features %lld exceeds what one CTA's shared memory holds "
                                       "(about 180000)", (long long)k_in);
    if (bt_device_count() <= device || device < 0)
        return set_error(BT_ERR_DEVICE, "bt_linear_create: no CUDA device %d", device);
    DeviceGuard guard(device);
    if (!guard.ok || !device_error_word(device))
        return set_error(BT_ERR_DEVICE, "bt_linear_create: cannot use device %d", device);

    bt_linear* lin = new (std::nothrow) bt_linear();
    if (!lin) return set_error(BT_ERR_NOMEM, "host allocation failed");
    lin->device = device;
    lin->w.n_out = n_out;
    lin->w.k_in = k_in;
    lin->w.n_bases = n_bases;
    lin->w.row_tiles = (n_out + kTileRows - 1) / kTileRows;
    lin->w.k_tiles = (k_in + kTileK - 1) / kTileK;
    for (int b = 0; b < n_bases; ++b) lin->scales[b] = scales_host[b];

    const size_t raw_bytes = (size_t)n_out * (size_t)(k_in / 4) * (size_t)n_bases;
    const size_t tile_bytes = (size_t)lin->w.basis_stride() * (size_t)n_bases;
    uint8_t* raw = nullptr;
    cudaError_t e = cudaMalloc(&lin->tiles, tile_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&raw, raw_bytes);
    if (e == cudaSuccess) e = cudaMemcpy(raw, packed_host, raw_bytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
        e = launch_retile(raw, n_out, k_in, n_bases, lin->tiles, lin->w.row_tiles, lin->w.k_tiles, 0);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaFree(raw);
    if (e != cudaSuccess) {
        cudaFree(lin->tiles);
        delete lin;
        return set_error(e == cudaErrorMemoryAllocation ? BT_ERR_NOMEM : BT_ERR_CUDA,
                         "bt_linear_create: %s", cudaGetErrorString(e));
    }
    lin->w.tiles = lin->tiles;
    {
        // one weight scale per (basis, half row tile); a plain BitLinear repeats scales[b]
        const size_t cnt = (size_t)n_bases * (size_t)lin->w.row_tiles * 2;
        float* host = new (std::nothrow) float[cnt];
        cudaError_t e2 = host ? cudaMalloc(&lin->scale_tiles, cnt * sizeof(float)) : cudaErrorMemoryAllocation;
        if (e2 == cudaSuccess) {
            for (int b = 0; b < n_bases; ++b)
                for (int64_t r = 0; r < lin->w.row_tiles * 2; ++r) host[(size_t)b * lin->w.row_tiles * 2 + r] = scales_host[b];
            e2 = cudaMemcpy(lin->scale_tiles, host, cnt * sizeof(float), cudaMemcpyHostToDevice);
        }
        delete[] host;
        if (e2 != cudaSuccess) {
            cudaFree(lin->tiles);
            cudaFree(lin->scale_tiles);
            delete lin;
            return set_error(BT_ERR_CUDA, "bt_linear_create: %s", cudaGetErrorString(e2));
        }
    }
    *out = lin;
    return BT_OK;
}

extern "C" bt_status bt_linear_destroy(bt_linear* lin) {
    if (!lin) return BT_OK;
    DeviceGuard guard(lin->device);
    cudaFree(lin->tiles);
    cudaFree(lin->scale_tiles);
    if (lin->own_ws) bt_workspace_destroy(lin->own_ws);
    delete lin;
    return BT_OK;
}

extern "C" bt_status bt_linear_dims(const bt_linear* lin, int64_t* n_out, int64_t* k_in, int* n_bases) {
    if (!lin) return set_error(BT_ERR_ARG, "bt_linear_dims: null handle");
    if (n_out) *n_out = lin->w.n_out;
    if (k_in) *k_in = lin->w.k_in;
    if (n_bases) *n_bases = lin->w.n_bases;
    return BT_OK;
}

// ---------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------
namespace {

struct WsPlan {
    int8_t* q;       // [m, k_pad]
    float* sx;       // [m]
    int32_t* qsum;   // [m]
    float* ytmp;     // [m, n] f32 (only when bf16 output needs several bases)
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

bt_status plan_workspace(bt_workspace* ws, int64_t m, int64_t k_pad, int64_t n, bool need_tmp,
                         WsPlan* p) {
    size_t off = 0;
    const size_t q_off = off;          off = align_up(off + (size_t)m * k_pad, 256);
    const size_t sx_off = off;         off = align_up(off + (size_t)m * 4, 256);
    const size_t qs_off = off;         off = align_up(off + (size_t)m * 4, 256);
    const size_t tmp_off = off;        if (need_tmp) off = align_up(off + (size_t)m * n * 4, 256);
    if (off > ws->bytes)
        return set_error(BT_ERR_NOMEM, "workspace of %zu bytes is too small: %zu needed for m=%lld",
                         ws->bytes, off, (long long)m);
    p->q = reinterpret_cast<int8_t*>(ws->base + q_off);
    p->sx = reinterpret_cast<float*>(ws->base + sx_off);
    p->qsum = reinterpret_cast<int32_t*>(ws->base + qs_off);
    p->ytmp = need_tmp ? reinterpret_cast<float*>(ws->base + tmp_off) : nullptr;
    return BT_OK;
}

bt_status resolve_workspace(bt_linear* lin, bt_workspace** ws) {
    if (*ws) {
        if ((*ws)->device != lin->device)
            return set_error(BT_ERR_DEVICE, "workspace is on device %d, layer on device %d",
                             (*ws)->device, lin->device);
        return BT_OK;
    }
    std::lock_guard<std::mutex> lock(lin->ws_mu);
    if (!lin->own_ws) {
        bt_status st = bt_workspace_create(&lin->own_ws, lin->device, 0);
        if (st != BT_OK) return st;
    }
    *ws = lin->own_ws;
    return BT_OK;
}

// Runs the product for all tokens and all bases on quantised activations.
bt_status run_product(bt_linear* lin, const WsPlan& p, int64_t m, void* out, bt_dtype out_dtype,
                      bool raw_i32, cudaStream_t stream) {
    const int sm = device_sm_count(lin->device);
    unsigned int* err = device_error_word(lin->device);
    const int64_t n = lin->w.n_out;
    const bool via_tmp = lin->w.n_bases > 1 && !raw_i32 && out_dtype == BT_BF16;
    const int epi = raw_i32 ? EPI_I32 : ((out_dtype == BT_BF16 && !via_tmp) ? EPI_BF16 : EPI_F32);
    BT_CUDA_TRY(linear_product(lin->dev(), p.q, lin->w.k_pad(), p.qsum, p.sx, m, via_tmp ? (void*)p.ytmp : out,
                               n, epi, err, sm, stream));
    if (via_tmp) {
        const int64_t total = m * n;
        int blocks = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
        cast_f32_to_bf16_kernel<<<blocks, 256, 0, stream>>>(p.ytmp, reinterpret_cast<__nv_bfloat16*>(out), total);
        BT_CUDA_TRY(cudaGetLastError());
    }
    return BT_OK;
}

}  // namespace

extern "C" bt_status bt_linear_forward(bt_linear* lin, bt_workspace* ws, const void* x_dev, int64_t m,
                                       int64_t x_k, bt_dtype x_dtype, void* y_dev, bt_dtype y_dtype,
                                       void* stream) {
    if (!lin) return set_error(BT_ERR_ARG, "bt_linear_forward: null handle");
    if (x_k != lin->w.k_in)  // wording of kernels/cpu.rs:22-30, kernels/cuda.rs:27-35
        return set_error(BT_ERR_SHAPE, "Shape mismatch: Input [%lld, %lld] vs Weight [%lld, %lld]",
                         (long long)m, (long long)x_k, (long long)lin->w.n_out, (long long)lin->w.k_in);
    if (m < 0) return set_error(BT_ERR_SHAPE, "bt_linear_forward: negative token count");
    if ((x_dtype != BT_F32 && x_dtype != BT_BF16) || (y_dtype != BT_F32 && y_dtype != BT_BF16))
        return set_error(BT_ERR_ARG, "bt_linear_forward: dtype must be BT_F32 or BT_BF16");
    if (m == 0) return BT_OK;
    if (!x_dev || !y_dev) return set_error(BT_ERR_ARG, "bt_linear_forward: null pointer");
    DeviceGuard guard(lin->device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "cannot select device %d", lin->device);
    bt_status st = resolve_workspace(lin, &ws);
    if (st != BT_OK) return st;
    WsPlan p;
    st = plan_workspace(ws, m, lin->w.k_pad(), lin->w.n_out, lin->w.n_bases > 1 && y_dtype == BT_BF16, &p);
    if (st != BT_OK) return st;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (m > 8 && !(lin->w.n_bases > 1 && y_dtype == BT_BF16) &&
        gemm_tc_act_bytes(m, lin->w.k_tiles) <= (size_t)m * lin->w.k_pad() + 256 * 1024 &&
        gemm_tc_act_bytes(m, lin->w.k_tiles) + 4096 <= ws->bytes) {
        // more than 8 tokens: tensor-core path (tcgen05), activations re-laid residue-split
        int8_t* qtc = reinterpret_cast<int8_t*>(ws->base);
        const size_t off = align_up(gemm_tc_act_bytes(m, lin->w.k_tiles), 256);
        if (off + (size_t)m * 8 + 512 <= ws->bytes) {
            float* sx = reinterpret_cast<float*>(ws->base + off);
            int32_t* qs = reinterpret_cast<int32_t*>(ws->base + off + align_up((size_t)m * 4, 256));
            BT_CUDA_TRY(launch_gemm_tc(lin->dev(), x_dev, lin->w.k_in, m, qtc, sx, qs, y_dev,
                                       lin->w.n_out, y_dtype == BT_BF16 ? EPI_BF16 : EPI_F32,
                                       device_error_word(lin->device), device_sm_count(lin->device), s, false, x_dtype));
            return BT_OK;
        }
    }
    BT_CUDA_TRY(launch_act_quant(x_dev, x_dtype, m, lin->w.k_in, p.q, lin->w.k_pad(), p.sx, p.qsum, s));
    return run_product(lin, p, m, y_dev, y_dtype, false, s);
}

__global__ void qsum_rows_kernel(const int8_t* __restrict__ q, int64_t stride, int64_t k,
                                 int32_t* __restrict__ qsum) {
    // one warp per token
    const int8_t* row = q + (int64_t)blockIdx.x * stride;
    int s = 0;
    for (int64_t c = threadIdx.x; c < k; c += 32) s += row[c];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) qsum[blockIdx.x] = s;
}

extern "C" bt_status bt_linear_forward_q(bt_linear* lin, bt_workspace* ws, const int8_t* q_dev,
                                         const float* sx_dev, int64_t m, void* out_dev,
                                         bt_dtype out_dtype, void* stream) {
    if (!lin || !q_dev || !out_dev) return set_error(BT_ERR_ARG, "bt_linear_forward_q: null pointer");
    if (out_dtype != BT_I32 && out_dtype != BT_F32)
        return set_error(BT_ERR_ARG, "bt_linear_forward_q: out_dtype must be BT_I32 or BT_F32");
    if (out_dtype == BT_F32 && !sx_dev) return set_error(BT_ERR_ARG, "bt_linear_forward_q: scales needed for BT_F32");
    if (m < 0) return set_error(BT_ERR_SHAPE, "bt_linear_forward_q: negative token count");
    if (m == 0) return BT_OK;
    DeviceGuard guard(lin->device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "cannot select device %d", lin->device);
    bt_status st = resolve_workspace(lin, &ws);
    if (st != BT_OK) return st;
    WsPlan p;
    st = plan_workspace(ws, m, lin->w.k_pad(), lin->w.n_out, false, &p);
    if (st != BT_OK) return st;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int64_t k = lin->w.k_in, kp = lin->w.k_pad();
    // stage into rows of k_pad bytes, zero beyond k
    if (kp != k) BT_CUDA_TRY(cudaMemsetAsync(p.q, 0, (size_t)m * kp, s));
    BT_CUDA_TRY(cudaMemcpy2DAsync(p.q, (size_t)kp, q_dev, (size_t)k, (size_t)k, (size_t)m,
                                  cudaMemcpyDeviceToDevice, s));
    qsum_rows_kernel<<<(unsigned)m, 32, 0, s>>>(p.q, kp, k, p.qsum);
    BT_CUDA_TRY(cudaGetLastError());
    if (sx_dev) BT_CUDA_TRY(cudaMemcpyAsync(p.sx, sx_dev, (size_t)m * 4, cudaMemcpyDeviceToDevice, s));
    return run_product(lin, p, m, out_dev, out_dtype, out_dtype == BT_I32, s);
}

extern "C" bt_status bt_linear_forward_host(bt_linear* lin, const float* x_host, int64_t m, int64_t x_k,
                                            float* y_host) {
    if (!lin || !x_host || !y_host) return set_error(BT_ERR_ARG, "bt_linear_forward_host: null pointer");
    if (x_k != lin->w.k_in)
        return set_error(BT_ERR_SHAPE, "Shape mismatch: Input [%lld, %lld] vs Weight [%lld, %lld]",
                         (long long)m, (long long)x_k, (long long)lin->w.n_out, (long long)lin->w.k_in);
    if (m <= 0) return m == 0 ? BT_OK : set_error(BT_ERR_SHAPE, "negative token count");
    DeviceGuard guard(lin->device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "cannot select device %d", lin->device);
    float *xd = nullptr, *yd = nullptr;
    const size_t xb = (size_t)m * x_k * 4, yb = (size_t)m * lin->w.n_out * 4;
    cudaError_t e = cudaMalloc(&xd, xb);
    if (e == cudaSuccess) e = cudaMalloc(&yd, yb);
    bt_status st = BT_OK;
    if (e == cudaSuccess) e = cudaMemcpy(xd, x_host, xb, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) st = bt_linear_forward(lin, nullptr, xd, m, x_k, BT_F32, yd, BT_F32, nullptr);
    if (e == cudaSuccess && st == BT_OK) e = cudaMemcpy(y_host, yd, yb, cudaMemcpyDeviceToHost);
    cudaFree(xd);
    cudaFree(yd);
    if (e != cudaSuccess) return set_error(BT_ERR_CUDA, "bt_linear_forward_host: %s", cudaGetErrorString(e));
    return st;
}

extern "C" bt_status bt_act_quant(const void* x_dev, bt_dtype x_dtype, int64_t m, int64_t k, int8_t* q_dev,
                                  float* s_dev, int32_t* qsum_dev, int device, void* stream) {
    if (!x_dev || !q_dev || !s_dev) return set_error(BT_ERR_ARG, "bt_act_quant: null pointer");
    if (x_dtype != BT_F32 && x_dtype != BT_BF16) return set_error(BT_ERR_ARG, "bt_act_quant: dtype must be BT_F32 or BT_BF16");
    if (m < 0 || k <= 0) return set_error(BT_ERR_SHAPE, "bt_act_quant: bad shape [%lld, %lld]", (long long)m, (long long)k);
    DeviceGuard guard(device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "cannot select device %d", device);
    BT_CUDA_TRY(launch_act_quant(x_dev, x_dtype, m, k, q_dev, k, s_dev, qsum_dev, reinterpret_cast<cudaStream_t>(stream)));
    return BT_OK;
}

extern "C" bt_status bt_linear_create_fused(bt_linear** out, const uint8_t* const* seg_packed_host,
                                            const int64_t* seg_rows, const float* seg_scales, int n_seg,
                                            int64_t k_in, int device) {
    if (!out) return set_error(BT_ERR_ARG, "bt_linear_create_fused: null out pointer");
    *out = nullptr;
    if (!seg_packed_host || !seg_rows || !seg_scales || n_seg < 1)
        return set_error(BT_ERR_ARG, "bt_linear_create_fused: null pointer or no segments");
    if (k_in <= 0 || k_in % 4 != 0)
        return set_error(BT_ERR_ALIGN, "bt_linear_create_fused: in_features %lld is not a multiple of 4", (long long)k_in);
    int64_t n_total = 0;
    for (int i = 0; i < n_seg; ++i) {
        if (!seg_packed_host[i] || seg_rows[i] <= 0 || seg_rows[i] % kTileRows != 0)
            return set_error(BT_ERR_ALIGN, "bt_linear_create_fused: segment %d has %lld rows (need a positive multiple of 16)",
                             i, (long long)seg_rows[i]);
        n_total += seg_rows[i];
    }
    const size_t row_bytes = (size_t)(k_in / 4);
    uint8_t* cat = new (std::nothrow) uint8_t[(size_t)n_total * row_bytes];
    if (!cat) return set_error(BT_ERR_NOMEM, "host allocation failed");
    size_t off = 0;
    for (int i = 0; i < n_seg; ++i) {
        memcpy(cat + off, seg_packed_host[i], (size_t)seg_rows[i] * row_bytes);
        off += (size_t)seg_rows[i] * row_bytes;
    }
    bt_linear* lin = nullptr;
    bt_status st = bt_linear_create(&lin, cat, n_total, k_in, 1, seg_scales, device);
    delete[] cat;
    if (st != BT_OK) return st;
    // overwrite the per-half-tile scales segment by segment
    float* host = new (std::nothrow) float[(size_t)lin->w.row_tiles * 2];
    if (!host) { bt_linear_destroy(lin); return set_error(BT_ERR_NOMEM, "host allocation failed"); }
    int64_t rt = 0;
    for (int i = 0; i < n_seg; ++i)
        for (int64_t r = 0; r < seg_rows[i] / kTileRows * 2; ++r) host[rt++] = seg_scales[i];
    DeviceGuard guard(device);
    cudaError_t e = cudaMemcpy(lin->scale_tiles, host, (size_t)lin->w.row_tiles * 2 * sizeof(float), cudaMemcpyHostToDevice);
    delete[] host;
    if (e != cudaSuccess) { bt_linear_destroy(lin); return set_error(BT_ERR_CUDA, "bt_linear_create_fused: %s", cudaGetErrorString(e)); }
    *out = lin;
    return BT_OK;
}

// ---------------------------------------------------------------------------------------
// forward without any allocation: scratch in a static device array
// ---------------------------------------------------------------------------------------
namespace {

constexpr size_t kNoAllocActBytes = BT_NOALLOC_MAX_ACT_BYTES;
constexpr size_t kNoAllocTailBytes = 1024;  // per-token scales and sums, 256-byte aligned slots

// Scratch of bt_linear_forward_noalloc: [quantised activations | scales | sums].  In host
// code this name is only a handle for cudaGetSymbolAddress; the kernels get the address
// that call returns.
static __device__ __align__(256) uint8_t g_noalloc_scratch[kNoAllocActBytes + kNoAllocTailBytes];

std::mutex g_noalloc_mu;
uint8_t* g_noalloc_ptr[kMaxDevices] = {nullptr};

// Once per device, with that device current: the array's address in device memory.
bt_status noalloc_scratch(int device, uint8_t** out) {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return set_error(BT_ERR_CUDA, "bt_linear_forward_noalloc: cudaGetSymbolAddress failed: %s",
                             cudaGetErrorString(e));
        g_noalloc_ptr[device] = static_cast<uint8_t*>(p);
    }
    *out = g_noalloc_ptr[device];
    return BT_OK;
}

}  // namespace

extern "C" bt_status bt_linear_forward_noalloc(bt_linear* lin, const void* x_dev, int64_t m, int64_t x_k,
                                               bt_dtype x_dtype, void* y_dev, bt_dtype y_dtype, void* stream) {
    if (!lin) return set_error(BT_ERR_ARG, "bt_linear_forward_noalloc: null handle");
    if (x_k != lin->w.k_in)
        return set_error(BT_ERR_SHAPE, "Shape mismatch: Input [%lld, %lld] vs Weight [%lld, %lld]",
                         (long long)m, (long long)x_k, (long long)lin->w.n_out, (long long)lin->w.k_in);
    if (m < 0) return set_error(BT_ERR_SHAPE, "bt_linear_forward_noalloc: negative token count");
    if ((x_dtype != BT_F32 && x_dtype != BT_BF16) || (y_dtype != BT_F32 && y_dtype != BT_BF16))
        return set_error(BT_ERR_ARG, "bt_linear_forward_noalloc: dtype must be BT_F32 or BT_BF16");
    if (m == 0) return BT_OK;
    if (!x_dev || !y_dev) return set_error(BT_ERR_ARG, "bt_linear_forward_noalloc: null pointer");
    const size_t act_bytes = (size_t)m * (size_t)lin->w.k_pad();
    if (m > 8 || act_bytes > kNoAllocActBytes)
        return set_error(BT_ERR_NOMEM,
                         "bt_linear_forward_noalloc: %lld tokens x %lld padded inputs = %zu bytes exceed the static "
                         "scratch (%zu bytes, at most 8 tokens); use bt_linear_forward with a workspace",
                         (long long)m, (long long)lin->w.k_pad(), act_bytes, kNoAllocActBytes);
    if (lin->w.n_bases > 1 && y_dtype == BT_BF16)
        return set_error(BT_ERR_ARG, "bt_linear_forward_noalloc: several bases need a BT_F32 output");
    DeviceGuard guard(lin->device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "cannot select device %d", lin->device);
    uint8_t* base = nullptr;
    bt_status st = noalloc_scratch(lin->device, &base);
    if (st != BT_OK) return st;
    WsPlan p;
    p.q = reinterpret_cast<int8_t*>(base);
    p.sx = reinterpret_cast<float*>(base + kNoAllocActBytes);
    p.qsum = reinterpret_cast<int32_t*>(base + kNoAllocActBytes + 256);
    p.ytmp = nullptr;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    BT_CUDA_TRY(launch_act_quant(x_dev, x_dtype, m, lin->w.k_in, p.q, lin->w.k_pad(), p.sx, p.qsum, s));
    return run_product(lin, p, m, y_dev, y_dtype, false, s);
}

namespace bt {

bt_status create_gate_up(bt_linear** out, const uint8_t* gate, const uint8_t* up, int64_t rows, int64_t k_in, int n_bases,
                         const float* gate_scales, const float* up_scales, int device) {
    if (!out || !gate || !up || !gate_scales || !up_scales) return set_error(BT_ERR_ARG, "create_gate_up: null pointer");
    if (rows <= 0 || rows % 8 != 0 || k_in <= 0 || k_in % 4 != 0)
        return set_error(BT_ERR_ALIGN, "create_gate_up: rows must be a multiple of 8 and in_features of 4");
    const size_t row_bytes = (size_t)(k_in / 4) * (size_t)n_bases;  // a row of the [rows, k_in/4, n_bases] layout
    uint8_t* cat = new (std::nothrow) uint8_t[(size_t)rows * 2 * row_bytes];
    if (!cat) return set_error(BT_ERR_NOMEM, "host allocation failed");
    for (int64_t t = 0; t < rows / 8; ++t) {
        memcpy(cat + (size_t)(16 * t) * row_bytes, gate + (size_t)(8 * t) * row_bytes, 8 * row_bytes);
        memcpy(cat + (size_t)(16 * t + 8) * row_bytes, up + (size_t)(8 * t) * row_bytes, 8 * row_bytes);
    }
    bt_linear* lin = nullptr;
    bt_status st = bt_linear_create(&lin, cat, rows * 2, k_in, n_bases, gate_scales, device);
    delete[] cat;
    if (st != BT_OK) return st;
    const size_t per_basis = (size_t)lin->w.row_tiles * 2, cnt = per_basis * (size_t)n_bases;
    float* host = new (std::nothrow) float[cnt];
    if (!host) { bt_linear_destroy(lin); return set_error(BT_ERR_NOMEM, "host allocation failed"); }
    for (int b = 0; b < n_bases; ++b)
        for (size_t i = 0; i < per_basis; ++i) host[(size_t)b * per_basis + i] = (i & 1) ? up_scales[b] : gate_scales[b];
    DeviceGuard guard(device);
    cudaError_t e = cudaMemcpy(lin->scale_tiles, host, cnt * sizeof(float), cudaMemcpyHostToDevice);
    delete[] host;
    if (e != cudaSuccess) { bt_linear_destroy(lin); return set_error(BT_ERR_CUDA, "create_gate_up: %s", cudaGetErrorString(e)); }
    *out = lin;
    return BT_OK;
}

}  // namespace bt
