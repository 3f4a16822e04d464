/*
 * CPU oracle for the BitLinear inference path of Bit-TTT-Engine.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It restates, in plain C, the
 * arithmetic of the reference's CPU kernels and layers so that the CUDA library can
 * be checked against it.  Only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark may load it; the CUDA library never does.
 *
 * Parity pin status:
 *   - pack/unpack (layout L1) and the 2-bit code table are pinned by the four
 *     known-answer tests of crates/rust_engine/src/kernels/packing.rs:156-261 and by
 *     fixtures generated from the reference's Python converter
 *     (tools/conversion/convert_llama_v2.py:28-72,111-151).
 *   - the ternary product (oracle_bitlinear_f32 / _i32 and the multi-basis sum) is
 *     pinned against the reference's own CUDA kernels (kernels/bit_op.cu:4-45,
 *     kernels/adaptive_bit_op.cu:74-161), compiled unchanged from the reference's
 *     source files by `make ref` into oracle/_ref/ and run in the GPU tests.
 *   - TTT, Q8 KV cache, RoPE, attention, RMSNorm, SwiGLU: the reference holds no
 *     value test for them and its Rust host code cannot be compiled here (no Rust
 *     toolchain), so for these functions PARITY IS UNPINNED: they follow the cited
 *     lines operation by operation, nothing more.
 *
 * Every function names the reference lines it follows (paths relative to the
 * reference project root).
 *
 * Reductions and transcendentals: the reference evaluates sums (RMSNorm mean, L2 norm,
 * matmul rows, softmax) and exp/cos/sin in f32 through candle ops whose evaluation order
 * and libm are not visible in its tree.  Here they are accumulated / evaluated in f64 and
 * rounded to f32 once: the correctly rounded value, within one f32 ulp of any f32
 * evaluation order and independent of how a checked implementation orders its sums.
 * Pointwise f32 operations keep the reference's order.  Built with -ffp-contract=off.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#define ORACLE_AVX2 1
#else
#define ORACLE_AVX2 0
#endif

#define EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------ */
/* 2-bit code table: 00 -> 0, 01 -> +1, 10 -> -1, 11 -> 0                                */
/* crates/rust_engine/src/kernels/packing.rs:9-13,120-124; kernels/cpu.rs:55-59          */
/* ------------------------------------------------------------------------------------ */
static inline int code_to_ternary(unsigned code) { return (int)(code & 1u) - (int)(code >> 1); }

EXPORT int oracle_has_avx2(void) { return ORACLE_AVX2; }

EXPORT int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* PackedTensor::pack  -- crates/rust_engine/src/kernels/packing.rs:50-105
 * scale = mean(|w|) + 1e-6 (:56-57); q = clamp(round(w/scale), -1, 1) (:60-65), round is
 * half-away-from-zero; code 1 if q > 0.5, 2 if q < -0.5, else 0 (:82-88); element i of
 * the FLATTENED tensor goes to bits 2*(i%4) of byte i/4 (:74-92).
 * The mean is accumulated in double and rounded to f32 once; candle's own f32
 * summation order is not visible from the reference tree, and the reference tests pin
 * the scale only to 1e-3.  Returns the scale; out must hold ceil(n/4) bytes. */
EXPORT float oracle_pack_l1(const float* w, int64_t n_elem, uint8_t* out) {
    double acc = 0.0;
    for (int64_t i = 0; i < n_elem; ++i) acc += fabs((double)w[i]);
    float mean = (float)(acc / (double)(n_elem > 0 ? n_elem : 1));
    float scale = mean + 1e-6f;
    if (n_elem <= 0) return scale;
    uint64_t nbytes = ((uint64_t)n_elem + 3u) / 4u;
    for (uint64_t i = 0; i < nbytes; ++i) out[i] = 0;
    for (int64_t i = 0; i < n_elem; ++i) {
        /* candle divides by (scale as f64) but the tensor stays f32: the divisor is the
         * f32 scale, the quotient an f32 (packing.rs:60). */
        float q = roundf(w[i] / scale);
        if (q > 1.0f) q = 1.0f;
        if (q < -1.0f) q = -1.0f;
        unsigned code = q > 0.5f ? 1u : (q < -0.5f ? 2u : 0u);
        out[i / 4] |= (uint8_t)(code << ((i % 4) * 2));
    }
    return scale;
}

/* PackedTensor::unpack -- crates/rust_engine/src/kernels/packing.rs:108-133 */
EXPORT void oracle_unpack_l1(const uint8_t* packed, int64_t n_elem, float scale, float* out) {
    for (int64_t i = 0; i < n_elem; ++i) {
        unsigned code = (packed[i / 4] >> ((i % 4) * 2)) & 3u;
        float v = code == 1 ? 1.0f : (code == 2 ? -1.0f : 0.0f);
        out[i] = v * scale;
    }
}

/* Converter-side 2-bit packing into layout [Out, In/4, NumBases]
 * tools/conversion/convert_llama_v2.py:111-151 -- bases are int8 in {-1,0,+1}, laid out
 * [NumBases, Out, In]; code = (v+3)%3; byte (o,q,b) = c0 | c1<<2 | c2<<4 | c3<<6. */
EXPORT void oracle_pack_l2(const int8_t* bases, int n_bases, int64_t n_out, int64_t k_in,
                           uint8_t* out) {
    int64_t kq = k_in / 4;
    for (int64_t o = 0; o < n_out; ++o)
        for (int64_t q = 0; q < kq; ++q)
            for (int b = 0; b < n_bases; ++b) {
                unsigned byte = 0;
                for (int r = 0; r < 4; ++r) {
                    int v = bases[((int64_t)b * n_out + o) * k_in + q * 4 + r];
                    unsigned code = (unsigned)((v + 3) % 3);
                    byte |= code << (2 * r);
                }
                out[(o * kq + q) * n_bases + b] = (uint8_t)byte;
            }
}

/* AdaptiveBitLinear::load dense reconstruction
 * crates/rust_engine/src/layers/adaptive_linear.rs:10-29 (LUT), :86-109 (index and sum):
 * W[o][4q+r] = sum_b LUT[packed[(o*K/4+q)*B+b]][r] * scales[b], accumulated in basis order. */
EXPORT void oracle_decode_l2(const uint8_t* packed, const float* scales, int n_bases,
                             int64_t n_out, int64_t k_in, float* w_out) {
    int64_t kq = k_in / 4;
    for (int64_t o = 0; o < n_out; ++o) {
        float* row = w_out + o * k_in;
        for (int64_t c = 0; c < k_in; ++c) row[c] = 0.0f;
        for (int b = 0; b < n_bases; ++b) {
            float s = scales[b];
            for (int64_t q = 0; q < kq; ++q) {
                unsigned byte = packed[(o * kq + q) * n_bases + b];
                for (int r = 0; r < 4; ++r)
                    row[q * 4 + r] += (float)code_to_ternary((byte >> (2 * r)) & 3u) * s;
            }
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* BitLinearCpu::forward -- crates/rust_engine/src/kernels/cpu.rs:17-127,134-239         */
/* ------------------------------------------------------------------------------------ */

/* compute_row_avx2 (cpu.rs:134-239): chunks of 32 inputs, 4 groups of 8; per group one
 * u16 of weights is expanded to 8 f32 coefficients (code&1)-(code>>1) (:205-212) and
 * fused-multiply-added into an 8-lane accumulator (:220); the 8 lanes are summed left
 * to right at the end (:236-238). */
static float row_chunks32(const float* x, const uint8_t* w, int64_t num_chunks) {
#if ORACLE_AVX2
    __m256 acc = _mm256_setzero_ps();
    for (int64_t c = 0; c < num_chunks; ++c) {
        for (int g = 0; g < 4; ++g) {
            uint16_t wv;
            memcpy(&wv, w, 2);
            w += 2;
            float coeffs[8];
            for (int b = 0; b < 8; ++b) {
                unsigned code = (wv >> (2 * b)) & 3u;
                coeffs[b] = (float)code_to_ternary(code);
            }
            __m256 wv8 = _mm256_loadu_ps(coeffs);
            __m256 xv8 = _mm256_loadu_ps(x);
            x += 8;
            acc = _mm256_fmadd_ps(xv8, wv8, acc);
        }
    }
    float lanes[8];
    _mm256_storeu_ps(lanes, acc);
#else
    float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int64_t c = 0; c < num_chunks; ++c) {
        for (int g = 0; g < 4; ++g) {
            unsigned wv = (unsigned)w[0] | ((unsigned)w[1] << 8);
            w += 2;
            for (int b = 0; b < 8; ++b) {
                unsigned code = (wv >> (2 * b)) & 3u;
                lanes[b] = fmaf(x[b], (float)code_to_ternary(code), lanes[b]);
            }
            x += 8;
        }
    }
#endif
    float s = 0.0f;
    for (int b = 0; b < 8; ++b) s += lanes[b];
    return s;
}

/* One output element, cpu.rs:77-123: AVX2 chunks, scalar remainder with LUT
 * [0,1,-1,0] (:59,105-122), then `sum * scale` (:123). */
static inline float bitlinear_one(const float* xrow, const uint8_t* wrow, int64_t k, float scale) {
    float sum = 0.0f;
    int64_t num_chunks = k / 32;
    sum += row_chunks32(xrow, wrow, num_chunks);
    for (int64_t l = num_chunks * 32; l < k; ++l) {
        unsigned code = (wrow[l / 4] >> ((l % 4) * 2)) & 3u;
        sum += xrow[l] * (float)code_to_ternary(code);
    }
    return sum * scale;
}

/* y[M,N] = scale * x[M,K] . T[N,K]^T, weight rows at stride ceil(K/4) bytes (cpu.rs:81).
 * Parallel over the M*N outputs like the reference's rayon par_iter_mut (cpu.rs:73-76).
 * Returns -1 on the reference's shape error (cpu.rs:22-30): never raised here because
 * the caller passes k for both; kept for interface symmetry. */
EXPORT int oracle_bitlinear_f32(const float* x, int64_t m, int64_t k, const uint8_t* packed,
                                int64_t n, float scale, float* y, int threads) {
    int64_t row_bytes = (k + 3) / 4;
    int64_t total = m * n;
    (void)threads;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : omp_get_max_threads())
#endif
    for (int64_t idx = 0; idx < total; ++idx) {
        int64_t i = idx / n, j = idx % n;
        y[idx] = bitlinear_one(x + i * k, packed + j * row_bytes, k, scale);
    }
    return 0;
}

/* Integer accumulators of the same product for int8 activations: acc[m,n] = sum_k q*t.
 * Equals what cpu.rs:73-124 computes with scale = 1 on the integer-valued f32 inputs
 * (every partial sum is an integer below 2^24, so f32 accumulation is exact). */
EXPORT void oracle_bitlinear_i32(const int8_t* q, int64_t m, int64_t k, const uint8_t* packed,
                                 int64_t n, int32_t* acc, int threads) {
    int64_t row_bytes = (k + 3) / 4;
    int64_t total = m * n;
    (void)threads;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : omp_get_max_threads())
#endif
    for (int64_t idx = 0; idx < total; ++idx) {
        int64_t i = idx / n, j = idx % n;
        const int8_t* qr = q + i * k;
        const uint8_t* wr = packed + j * row_bytes;
        int32_t s = 0;
        for (int64_t l = 0; l < k; ++l)
            s += (int32_t)qr[l] * code_to_ternary((wr[l / 4] >> ((l % 4) * 2)) & 3u);
        acc[idx] = s;
    }
}

/* Per-token absmax int8 quantiser placed in front of the ternary product.  The
 * reference has no such stage on this path; the definition is the BitNet b1.58 one, in the
 * spirit of the reference's only absmax quantiser (crates/rust_engine/src/layers/
 * kv_cache.rs:95-119) without the +128 zero-point:
 *   amax = max|x|;  q = clamp(round(x * (127/amax)), -127, 127)  (round half away from zero,
 *   the multiplier 127/amax computed once per token in f32);  dequantisation scale
 *   s = amax/127;  an all-zero row gives s = 0, q = 0 (the reference would give NaN).
 * Also returns sum_k q per token, which the CUDA kernels use internally. */
EXPORT void oracle_act_quant(const float* x, int64_t m, int64_t k, int8_t* q, float* s_out,
                             int32_t* qsum_out) {
    for (int64_t i = 0; i < m; ++i) {
        const float* xr = x + i * k;
        float amax = 0.0f;
        for (int64_t l = 0; l < k; ++l) {
            float a = fabsf(xr[l]);
            if (a > amax) amax = a;
        }
        float s = amax / 127.0f;
        float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
        int32_t sum = 0;
        for (int64_t l = 0; l < k; ++l) {
            float r = 0.0f;
            if (amax > 0.0f) {
                r = roundf(xr[l] * inv);
                if (r > 127.0f) r = 127.0f;
                if (r < -127.0f) r = -127.0f;
            }
            q[i * k + l] = (int8_t)r;
            sum += (int32_t)r;
        }
        s_out[i] = s;
        if (qsum_out) qsum_out[i] = sum;
    }
}

/* Quantised BitLinear forward: act_quant -> BitLinearCpu::forward on the integer-valued
 * activations (cpu.rs:73-124, `sum * scale` at :123) -> times the per-token scale.
 * y = ((float)acc * s_w) * s_x[m]; with n_bases > 1 (layout [N,K/4,B],
 * adaptive_linear.rs:99) y = sum_b ((float)acc_b * scales[b]) * s_x[m] in basis order. */
EXPORT void oracle_bitlinear_q(const float* x, int64_t m, int64_t k, const uint8_t* packed,
                               int n_bases, const float* scales, int64_t n, float* y,
                               int threads) {
    int8_t* q = (int8_t*)malloc((size_t)(m * k));
    float* sx = (float*)malloc(sizeof(float) * (size_t)m);
    oracle_act_quant(x, m, k, q, sx, NULL);
    int64_t kq = k / 4;
    int64_t total = m * n;
    (void)threads;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : omp_get_max_threads())
#endif
    for (int64_t idx = 0; idx < total; ++idx) {
        int64_t i = idx / n, j = idx % n;
        const int8_t* qr = q + i * k;
        float out = 0.0f;
        for (int b = 0; b < n_bases; ++b) {
            int32_t s = 0;
            for (int64_t c = 0; c < kq; ++c) {
                unsigned byte = packed[(j * kq + c) * n_bases + b];
                for (int r = 0; r < 4; ++r)
                    s += (int32_t)qr[c * 4 + r] * code_to_ternary((byte >> (2 * r)) & 3u);
            }
            out += ((float)s * scales[b]) * sx[i];
        }
        y[idx] = out;
    }
    free(q);
    free(sx);
}

/* ------------------------------------------------------------------------------------ */
/* Glue layers                                                                           */
/* ------------------------------------------------------------------------------------ */

/* RMSNorm::forward -- crates/rust_engine/src/layers/rms_norm.rs:33-56:
 * y = x / sqrt(mean(x^2) + eps) * w, all f32, eps inside the sqrt. */
EXPORT void oracle_rmsnorm(const float* x, int64_t m, int64_t h, const float* w, float eps,
                           float* y) {
    for (int64_t i = 0; i < m; ++i) {
        const float* xr = x + i * h;
        double ss = 0.0;
        for (int64_t c = 0; c < h; ++c) ss += (double)xr[c] * (double)xr[c];
        float denom = sqrtf((float)(ss / (double)h) + eps);
        for (int64_t c = 0; c < h; ++c) y[i * h + c] = (xr[c] / denom) * w[c];
    }
}

/* silu(g) * u -- crates/rust_engine/src/layers/swiglu.rs:31-33 (candle_nn::ops::silu =
 * x / (1 + exp(-x))). */
EXPORT void oracle_silu_mul(const float* g, const float* u, int64_t n, float* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = (g[i] / (1.0f + (float)exp(-(double)g[i]))) * u[i];
}

/* ------------------------------------------------------------------------------------ */
/* TTT fast-weight layer inner step (without the down/up projections)                    */
/* ------------------------------------------------------------------------------------ */

/* TTTLayer::forward_update -- crates/rust_engine/src/layers/ttt.rs:52-68.
 * feat[d] -> fhat = feat/(sqrt(sum feat^2) + 1e-6); z = W fhat; diff = z - fhat;
 * W' = W - lr * diff fhat^T.  W is d x d row-major, updated in place; z_out gets the
 * prediction made with the OLD W (:58-59,71). */
EXPORT void oracle_ttt_step(float* w, const float* feat, int64_t d, float lr, float* z_out) {
    float* fh = (float*)malloc(sizeof(float) * (size_t)d * 2);
    float* diff = fh + d;
    double ss = 0.0;
    for (int64_t c = 0; c < d; ++c) ss += (double)feat[c] * (double)feat[c];
    float nrm = sqrtf((float)ss) + 1e-6f;
    for (int64_t c = 0; c < d; ++c) fh[c] = feat[c] / nrm;
    for (int64_t a = 0; a < d; ++a) {
        double acc = 0.0;
        for (int64_t c = 0; c < d; ++c) acc += (double)w[a * d + c] * (double)fh[c];
        float s = (float)acc;
        z_out[a] = s;
        diff[a] = s - fh[a];
    }
    for (int64_t a = 0; a < d; ++a)
        for (int64_t c = 0; c < d; ++c) w[a * d + c] -= (diff[a] * fh[c]) * lr;
    free(fh);
}

/* TTTLayer::forward_chunkwise inner loop -- crates/rust_engine/src/layers/ttt.rs:88-113.
 * feats: T x d.  All rows are normalised first (:88-90); per chunk of `chunk` rows X:
 * Z = X W^T (:103-106); D = Z - X; G = D^T X (:107-109); W -= lr*G once per chunk (:111).
 * z_out: T x d. */
EXPORT void oracle_ttt_chunk(float* w, const float* feats, int64_t t_len, int64_t d, float lr,
                             int64_t chunk, float* z_out) {
    float* xh = (float*)malloc(sizeof(float) * (size_t)(t_len * d));
    float* g = (float*)malloc(sizeof(float) * (size_t)(d * d));
    for (int64_t t = 0; t < t_len; ++t) {
        double ss = 0.0;
        for (int64_t c = 0; c < d; ++c) ss += (double)feats[t * d + c] * (double)feats[t * d + c];
        float nrm = sqrtf((float)ss) + 1e-6f;
        for (int64_t c = 0; c < d; ++c) xh[t * d + c] = feats[t * d + c] / nrm;
    }
    for (int64_t start = 0; start < t_len; start += chunk) {
        int64_t len = t_len - start < chunk ? t_len - start : chunk;
        for (int64_t t = start; t < start + len; ++t)
            for (int64_t a = 0; a < d; ++a) {
                double acc = 0.0;
                for (int64_t c = 0; c < d; ++c) acc += (double)w[a * d + c] * (double)xh[t * d + c];
                z_out[t * d + a] = (float)acc;
            }
        for (int64_t a = 0; a < d; ++a)
            for (int64_t c = 0; c < d; ++c) {
                double acc = 0.0;
                for (int64_t t = start; t < start + len; ++t)
                    acc += (double)(z_out[t * d + a] - xh[t * d + a]) * (double)xh[t * d + c];
                g[a * d + c] = (float)acc;
            }
        for (int64_t i = 0; i < d * d; ++i) w[i] -= g[i] * lr;
    }
    free(xh);
    free(g);
}

/* ------------------------------------------------------------------------------------ */
/* Q8 KV cache, RoPE, attention                                                          */
/* ------------------------------------------------------------------------------------ */

/* QuantizedKVCache::quantize_q8 -- crates/rust_engine/src/layers/kv_cache.rs:95-119:
 * per row of `hd` values: s = max|x|/127; q = u8(round(x/s) + 128).  s == 0 -> q = 128
 * (the reference divides 0/0 there). */
EXPORT void oracle_kv_quant(const float* x, int64_t rows, int64_t hd, uint8_t* q, float* s_out) {
    for (int64_t i = 0; i < rows; ++i) {
        float amax = 0.0f;
        for (int64_t c = 0; c < hd; ++c) {
            float a = fabsf(x[i * hd + c]);
            if (a > amax) amax = a;
        }
        float s = amax / 127.0f;
        for (int64_t c = 0; c < hd; ++c) {
            float r = s > 0.0f ? roundf(x[i * hd + c] / s) : 0.0f;
            float sh = r + 128.0f;
            if (sh < 0.0f) sh = 0.0f;
            if (sh > 255.0f) sh = 255.0f;
            q[i * hd + c] = (uint8_t)sh;
        }
        s_out[i] = s;
    }
}

/* dequantize_q8 -- kv_cache.rs:122-128: (f32(q) - 128) * s */
EXPORT void oracle_kv_dequant(const uint8_t* q, const float* s, int64_t rows, int64_t hd,
                              float* out) {
    for (int64_t i = 0; i < rows; ++i)
        for (int64_t c = 0; c < hd; ++c) out[i * hd + c] = ((float)q[i * hd + c] - 128.0f) * s[i];
}

/* RotaryEmbedding::new + apply -- crates/rust_engine/src/layers/attention.rs:15-41,45-84.
 * inv_freq[i] = (1/theta^(2i/hd)) evaluated in f64 and cast to f32 (:19-22); freq =
 * f32(pos) * inv_freq (f32 product, :30); cos/sin of that f32 (:33-34); halves x1, x2:
 * out = [x1*cos - x2*sin, x1*sin + x2*cos] (:79-83).  x: rows x hd, every row rotated
 * at the same position `pos`, in place. */
EXPORT void oracle_rope(float* x, int64_t rows, int64_t hd, int64_t pos, double theta) {
    int64_t half = hd / 2;
    for (int64_t i = 0; i < half; ++i) {
        float inv = (float)(1.0 / pow(theta, (double)(2 * i) / (double)hd));
        float fr = (float)pos * inv;
        float c = (float)cos((double)fr), s = (float)sin((double)fr);
        for (int64_t r = 0; r < rows; ++r) {
            float x1 = x[r * hd + i], x2 = x[r * hd + half + i];
            x[r * hd + i] = x1 * c - x2 * s;
            x[r * hd + half + i] = x1 * s + x2 * c;
        }
    }
}

/* Single-query attention over a dequantised cache, one sequence.
 * BitAttention::forward -- crates/rust_engine/src/layers/attention.rs:198-217 with
 * seq_len == 1 (no mask, :242-245): scores = (q.k) * (1/sqrt(hd)) (:202); softmax over
 * keys (:214); out = p.v (:217).  Heads h use kv head h / (n_heads/n_kv) (repeat_kv,
 * :228-239).  q: n_heads x hd (already rotated); k, v: n_kv x T x hd (dequantised);
 * out: n_heads x hd. */
EXPORT void oracle_attn_decode(const float* q, const float* k, const float* v, int64_t n_heads,
                               int64_t n_kv, int64_t t_len, int64_t hd, float* out) {
    int64_t rep = n_heads / n_kv;
    float scaling = (float)(1.0 / sqrt((double)hd));
    float* sc = (float*)malloc(sizeof(float) * (size_t)t_len);
    double* pr = (double*)malloc(sizeof(double) * (size_t)t_len);
    for (int64_t h = 0; h < n_heads; ++h) {
        const float* kh = k + (h / rep) * t_len * hd;
        const float* vh = v + (h / rep) * t_len * hd;
        float mx = -INFINITY;
        for (int64_t t = 0; t < t_len; ++t) {
            double acc = 0.0;
            for (int64_t c = 0; c < hd; ++c) acc += (double)q[h * hd + c] * (double)kh[t * hd + c];
            float s = (float)acc * scaling;
            sc[t] = s;
            if (s > mx) mx = s;
        }
        double den = 0.0;
        for (int64_t t = 0; t < t_len; ++t) {
            pr[t] = exp((double)sc[t] - (double)mx);
            den += pr[t];
        }
        for (int64_t c = 0; c < hd; ++c) {
            double acc = 0.0;
            for (int64_t t = 0; t < t_len; ++t) acc += pr[t] * (double)vh[t * hd + c];
            out[h * hd + c] = (float)(acc / den);
        }
    }
    free(sc);
    free(pr);
}

/* Dense f32 linear without bias: y[M,N] = x[M,K] . W[N,K]^T -- the lm_head
 * (candle_nn::Linear, crates/rust_engine/src/model/llama.rs:23,266). */
EXPORT void oracle_dense_linear(const float* x, int64_t m, int64_t k, const float* w, int64_t n,
                                float* y, int threads) {
    int64_t total = m * n;
    (void)threads;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : omp_get_max_threads())
#endif
    for (int64_t idx = 0; idx < total; ++idx) {
        int64_t i = idx / n, j = idx % n;
        float s = 0.0f;
        for (int64_t c = 0; c < k; ++c) s += x[i * k + c] * w[j * k + c];
        y[idx] = s;
    }
}
