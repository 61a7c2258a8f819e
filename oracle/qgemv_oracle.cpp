// CPU oracle for the weight-only quantized GEMV path.  TEST INFRASTRUCTURE ONLY.
//
// This file is the checker the GPU library is compared against.  Nothing in the
// shipped library links, imports or calls it; only the test-suite, the smoke
// check and the CPU-baseline / reference legs of the benchmark may load it.
//
// Parity status: PARITY UNPINNED at the reference boundary.  The registry
// project (crit-labs/crit-hub) ships no implementation and no test vectors of
// this arithmetic: its engine cards only name the formats ("NVFP4 E2M1 with
// E4M3 group scales", tools/fixtures/engines/crit-labs/mtp-adaptive-width/card.yaml:74;
// "FP8 per-channel ... output head", tools/fixtures/engines/crit-labs/mtp4-nvfp4-mma/card.yaml:74;
// "quantized-projections ... decode rows on mma-rows and decode-gemv",
// engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:77) and keep the kernels in
// crit-labs/crit-engines @ dc41ff0d8f6f2dcbcf54fc87ede71232cc42046e and
// @ 53e4423ba6f0704a0d8862e2c15add650edef6a9, which are not vendored.  What is
// restated here is therefore the public definition of the formats:
//   * E2M1 (OCP MX FP4): 1 sign, 2 exponent (bias 1), 1 mantissa bit;
//     magnitudes {0, 0.5, 1, 1.5, 2, 3, 4, 6}.
//   * E4M3 "fn" (OCP FP8): 1-4-3, bias 7, subnormals m * 2^-9, max 448,
//     0x7F / 0xFF are NaN, no infinities.
//   * bfloat16: upper 16 bits of IEEE binary32, round to nearest even.
//   * NVFP4 tensor: E2M1 codes, one E4M3 scale per 16 consecutive K elements,
//     one fp32 per-tensor scale.
// The codecs are cross-checked in the tests against ml_dtypes and torch, and
// against committed exhaustive tables (tests/golden).
//
// Canonical (unpacked) storage used by every function below:
//   NVFP4: codes  u8 [N][K/2]  (low nibble = even k, high nibble = odd k)
//          scales u8 [N][K/16] (E4M3), tensor_scale fp32
//   FP8:   codes  u8 [N][K]    (E4M3), channel_scale fp32 [N]
//   x:     bf16 bit patterns u16 [B][K]
//
// Dequantisation rule (the "bit-exact" contract):
//   NVFP4: w = fp32( e2m1(code) * e4m3(scale) )  -- exact, <= 6 significant bits
//          w = fp32( w * tensor_scale )           -- one rounding, RN-even
//   FP8:   w = fp32( fp32(e4m3(code)) * channel_scale[n] )
// GEMV oracle: y[b][n] = sum_k double(w[n][k]) * double(x[b][k]), k ascending.
//
// Build: g++ -O2 -fopenmp -ffp-contract=off -shared -fPIC (see oracle/build.py).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <limits>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline float bits_to_f32(uint32_t u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint32_t f32_to_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}

// E2M1: s | e e | m.  e == 0 is subnormal: value = m * 0.5.
inline float e2m1_decode(uint32_t code) {
    const uint32_t s = (code >> 3) & 1u, e = (code >> 1) & 3u, m = code & 1u;
    float mag;
    if (e == 0) {
        mag = 0.5f * float(m);
    } else {
        mag = std::ldexp(1.0f + 0.5f * float(m), int(e) - 1);
    }
    return s ? -mag : mag;
}

// E4M3fn: s | eeee | mmm, bias 7.
inline float e4m3_decode(uint32_t b) {
    const uint32_t s = (b >> 7) & 1u, e = (b >> 3) & 15u, m = b & 7u;
    float mag;
    if (e == 15 && m == 7) {
        return std::numeric_limits<float>::quiet_NaN();
    } else if (e == 0) {
        mag = std::ldexp(float(m), -9);
    } else {
        mag = std::ldexp(1.0f + float(m) / 8.0f, int(e) - 7);
    }
    return s ? -mag : mag;
}

// fp32 -> E4M3fn, round to nearest even, saturating to +-448, NaN -> 0x7F|sign.
inline uint8_t e4m3_encode(float f) {
    const uint32_t u = f32_to_bits(f);
    const uint8_t sign = uint8_t((u >> 24) & 0x80u);
    if (std::isnan(f)) return uint8_t(sign | 0x7Fu);
    const float a = std::fabs(f);
    if (a >= 464.0f) return uint8_t(sign | 0x7Eu);  // above the 448/480 midpoint: saturate
    if (a == 0.0f) return sign;
    int ex;
    (void)std::frexp(a, &ex);  // a = fr * 2^ex, fr in [0.5, 1)
    int e = ex - 1;            // a = 1.xxx * 2^e
    if (e < -6) e = -6;        // subnormal range shares the 2^-6 exponent
    // quantum = 2^(e-3); q = a / quantum rounded to nearest even integer
    const float q = std::nearbyint(std::ldexp(a, 3 - e));  // default rounding mode: RN-even
    int qi = int(q);
    if (e == -6 && qi < 8) {
        return uint8_t(sign | uint8_t(qi));  // subnormal (or zero)
    }
    if (qi == 16) {  // mantissa overflowed into the next binade
        qi = 8;
        e += 1;
    }
    int be = e + 7;
    if (be > 15 || (be == 15 && (qi - 8) == 7)) return uint8_t(sign | 0x7Eu);
    return uint8_t(sign | uint8_t(be << 3) | uint8_t(qi - 8));
}

inline float bf16_decode(uint16_t h) { return bits_to_f32(uint32_t(h) << 16); }

// fp32 -> bf16 bit pattern, round to nearest even; NaN stays a quiet NaN.
inline uint16_t bf16_encode(float f) {
    uint32_t u = f32_to_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((u >> 16) | 0x0040u);
    const uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return uint16_t(u >> 16);
}

// fp32 -> E2M1 code, round to nearest, ties to the even mantissa bit, saturating at +-6; the sign bit
// of the input is kept (so -0 and tiny negatives give code 8).  The grid is 0, .5, 1, 1.5, 2, 3, 4, 6.
inline uint8_t e2m1_encode(float f) {
    const uint8_t sign = std::signbit(f) ? 8u : 0u;
    const float a = std::fabs(f);
    uint8_t c;
    if (a <= 0.25f) c = 0;          // tie 0.25 -> 0   (mantissa 0)
    else if (a < 0.75f) c = 1;      // 0.5
    else if (a <= 1.25f) c = 2;     // ties 0.75 -> 1, 1.25 -> 1
    else if (a < 1.75f) c = 3;      // 1.5
    else if (a <= 2.5f) c = 4;      // ties 1.75 -> 2, 2.5 -> 2
    else if (a < 3.5f) c = 5;       // 3
    else if (a <= 5.0f) c = 6;      // ties 3.5 -> 4, 5 -> 4
    else c = 7;                     // 6 (saturating)
    return uint8_t(sign | c);
}

inline float nvfp4_weight(uint32_t code, uint32_t scale_byte, float tensor_scale) {
    volatile float t = e2m1_decode(code) * e4m3_decode(scale_byte);  // exact product
    volatile float w = t * tensor_scale;                             // single fp32 rounding
    return w;
}

inline float fp8_weight(uint32_t code, float channel_scale) {
    volatile float w = e4m3_decode(code) * channel_scale;
    return w;
}

}  // namespace

extern "C" {

// ---- codecs ---------------------------------------------------------------------------------
float orc_e2m1_decode(uint32_t code) { return e2m1_decode(code & 15u); }
float orc_e4m3_decode(uint32_t byte) { return e4m3_decode(byte & 255u); }
uint32_t orc_e4m3_encode(float f) { return e4m3_encode(f); }
float orc_bf16_decode(uint32_t h) { return bf16_decode(uint16_t(h)); }
uint32_t orc_bf16_encode(float f) { return bf16_encode(f); }

void orc_e4m3_encode_array(const float* in, uint8_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = e4m3_encode(in[i]);
}
void orc_bf16_encode_array(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = bf16_encode(in[i]);
}
void orc_bf16_decode_array(const uint16_t* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = bf16_decode(in[i]);
}

// ---- dequantisation to fp32 [N][K] ----------------------------------------------------------
void orc_dequant_nvfp4(const uint8_t* codes, const uint8_t* scales, float tensor_scale, int64_t N,
                       int64_t K, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* c = codes + n * (K / 2);
        const uint8_t* s = scales + n * (K / 16);
        float* o = out + n * K;
        for (int64_t k = 0; k < K; ++k) {
            const uint32_t byte = c[k >> 1];
            const uint32_t code = (k & 1) ? (byte >> 4) : (byte & 15u);
            o[k] = nvfp4_weight(code, s[k >> 4], tensor_scale);
        }
    }
}

void orc_dequant_fp8(const uint8_t* codes, const float* channel_scale, int64_t N, int64_t K,
                     float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t k = 0; k < K; ++k) out[n * K + k] = fp8_weight(codes[n * K + k], channel_scale[n]);
    }
}

// ---- fp64-accumulated GEMV / skinny GEMM oracle: y f64 [B][N] -------------------------------
void orc_gemv_nvfp4_f64(const uint8_t* codes, const uint8_t* scales, float tensor_scale, int64_t N,
                        int64_t K, const uint16_t* x, int64_t B, double* y) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* c = codes + n * (K / 2);
        const uint8_t* s = scales + n * (K / 16);
        for (int64_t b = 0; b < B; ++b) {
            const uint16_t* xb = x + b * K;
            double acc = 0.0;
            for (int64_t k = 0; k < K; ++k) {
                const uint32_t byte = c[k >> 1];
                const uint32_t code = (k & 1) ? (byte >> 4) : (byte & 15u);
                acc += double(nvfp4_weight(code, s[k >> 4], tensor_scale)) * double(bf16_decode(xb[k]));
            }
            y[b * N + n] = acc;
        }
    }
}

void orc_gemv_fp8_f64(const uint8_t* codes, const float* channel_scale, int64_t N, int64_t K,
                      const uint16_t* x, int64_t B, double* y) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t b = 0; b < B; ++b) {
            const uint16_t* xb = x + b * K;
            double acc = 0.0;
            for (int64_t k = 0; k < K; ++k)
                acc += double(fp8_weight(codes[n * K + k], channel_scale[n])) * double(bf16_decode(xb[k]));
            y[b * N + n] = acc;
        }
    }
}

// ---- fast CPU GEMV: fp32 accumulate, OpenMP over rows (the timed CPU baseline) --------------
// Returns the number of OpenMP threads used.  y is fp32 [B][N].
int orc_gemv_nvfp4_fast(const uint8_t* codes, const uint8_t* scales, float tensor_scale, int64_t N,
                        int64_t K, const uint16_t* x, int64_t B, float* y) {
    float lut[256][2];
    for (int i = 0; i < 256; ++i) {
        lut[i][0] = e2m1_decode(i & 15);
        lut[i][1] = e2m1_decode(i >> 4);
    }
    float slut[256];
    for (int i = 0; i < 256; ++i) slut[i] = e4m3_decode(i);
    float* xf = new float[B * K];
    for (int64_t i = 0; i < B * K; ++i) xf[i] = bf16_decode(x[i]);
    int threads = 1;
#ifdef _OPENMP
    threads = omp_get_max_threads();
#endif
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* c = codes + n * (K / 2);
        const uint8_t* s = scales + n * (K / 16);
        for (int64_t b = 0; b < B; ++b) {
            const float* xb = xf + b * K;
            float acc = 0.0f;
            for (int64_t kb = 0; kb < K / 16; ++kb) {
                float part = 0.0f;
                const uint8_t* cb = c + kb * 8;
                const float* xk = xb + kb * 16;
                for (int j = 0; j < 8; ++j) {
                    part += lut[cb[j]][0] * xk[2 * j];
                    part += lut[cb[j]][1] * xk[2 * j + 1];
                }
                acc += part * slut[s[kb]];
            }
            y[b * N + n] = acc * tensor_scale;
        }
    }
    delete[] xf;
    return threads;
}

int orc_gemv_fp8_fast(const uint8_t* codes, const float* channel_scale, int64_t N, int64_t K,
                      const uint16_t* x, int64_t B, float* y) {
    float slut[256];
    for (int i = 0; i < 256; ++i) slut[i] = e4m3_decode(i);
    float* xf = new float[B * K];
    for (int64_t i = 0; i < B * K; ++i) xf[i] = bf16_decode(x[i]);
    int threads = 1;
#ifdef _OPENMP
    threads = omp_get_max_threads();
#endif
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* c = codes + n * K;
        for (int64_t b = 0; b < B; ++b) {
            const float* xb = xf + b * K;
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k) acc += slut[c[k]] * xb[k];
            y[b * N + n] = acc * channel_scale[n];
        }
    }
    delete[] xf;
    return threads;
}

// ---- MoE oracle -----------------------------------------------------------------------------
// For every (token t, slot j): out[t*topk + j][:] = W[expert_ids[t][j]] . x[xrow][:], fp64,
// where xrow = t (shared input, gate/up stage) or t*topk + j (per-slot input, down stage).
// Expert e's canonical tensors are stacked: codes [E][N][K/2], scales [E][N][K/16], ts [E].
void orc_moe_gemv_nvfp4_f64(const uint8_t* codes, const uint8_t* scales, const float* tensor_scales,
                            int64_t N, int64_t K, const int32_t* expert_ids, int64_t T, int64_t topk,
                            const uint16_t* x, int per_slot_input, double* out) {
    const int64_t cstride = N * (K / 2), sstride = N * (K / 16);
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t j = 0; j < topk; ++j) {
            const int64_t e = expert_ids[t * topk + j];
            const int64_t xrow = per_slot_input ? (t * topk + j) : t;
            orc_gemv_nvfp4_f64(codes + e * cstride, scales + e * sstride, tensor_scales[e], N, K,
                               x + xrow * K, 1, out + (t * topk + j) * N);
        }
    }
}

// ---- activations quantised to NVFP4 (the A4 mode of the skinny GEMM) -----------------------------
// The quantiser, stated once so that the device kernel can be held to it bit for bit.  Per row m of
// bf16 activations (K a multiple of 16), all arithmetic in fp32 with round-to-nearest-even:
//   amax = max |x[m][:]|;  g = amax == 0 ? 1 : amax / 2688           (2688 = 6 * 448)
//   per block of 16:  a = max |x| in the block;  s = E4M3(a / (6 * g))   (saturating)
//                     t = decode(s) * g;  code[k] = t == 0 ? 0 : E2M1(x[k] / t)   (saturating, sign kept)
// The dequantised activation is decode(code) * decode(s) * g.
void orc_quantize_a4(const uint16_t* x, int64_t M, int64_t K, uint8_t* codes, uint8_t* scales, float* g_out) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        const uint16_t* xr = x + m * K;
        float amax = 0.f;
        for (int64_t k = 0; k < K; ++k) amax = std::max(amax, std::fabs(bf16_decode(xr[k])));
        volatile float g = amax == 0.f ? 1.0f : amax / 2688.0f;
        g_out[m] = g;
        volatile float d6 = 6.0f * g;
        for (int64_t kb = 0; kb < K / 16; ++kb) {
            float a = 0.f;
            for (int e = 0; e < 16; ++e) a = std::max(a, std::fabs(bf16_decode(xr[kb * 16 + e])));
            volatile float sf = a / d6;
            const uint8_t sb = e4m3_encode(sf);
            scales[m * (K / 16) + kb] = sb;
            volatile float t = e4m3_decode(sb) * g;
            for (int e = 0; e < 16; e += 2) {
                uint8_t c[2] = {0, 0};
                if (t != 0.f) {
                    for (int z = 0; z < 2; ++z) {
                        volatile float q = bf16_decode(xr[kb * 16 + e + z]) / t;
                        c[z] = e2m1_encode(q);
                    }
                }
                codes[m * (K / 2) + (kb * 16 + e) / 2] = uint8_t(c[0] | (c[1] << 4));
            }
        }
    }
}

// Y[M][N] in fp64 from NVFP4 weights and NVFP4-quantised activations (codes, block scales, row scales).
void orc_gemm_nvfp4_a4_f64(const uint8_t* wcodes, const uint8_t* wscales, float tensor_scale, int64_t N, int64_t K,
                           const uint8_t* xcodes, const uint8_t* xscales, const float* g, int64_t M, double* y) {
    std::vector<double> xq(size_t(M) * size_t(K));
    for (int64_t m = 0; m < M; ++m)
        for (int64_t k = 0; k < K; ++k) {
            const uint8_t byte = xcodes[m * (K / 2) + k / 2];
            const uint32_t code = (k & 1) ? (byte >> 4) : (byte & 15u);
            xq[size_t(m * K + k)] = double(e2m1_decode(code)) * double(e4m3_decode(xscales[m * (K / 16) + k / 16])) * double(g[m]);
        }
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        std::vector<double> w(static_cast<size_t>(K));
        for (int64_t k = 0; k < K; ++k) {
            const uint8_t byte = wcodes[n * (K / 2) + k / 2];
            const uint32_t code = (k & 1) ? (byte >> 4) : (byte & 15u);
            w[size_t(k)] = double(e2m1_decode(code)) * double(e4m3_decode(wscales[n * (K / 16) + k / 16]));
        }
        for (int64_t m = 0; m < M; ++m) {
            double acc = 0.0;
            for (int64_t k = 0; k < K; ++k) acc += w[size_t(k)] * xq[size_t(m * K + k)];
            y[m * N + n] = acc * double(tensor_scale);
        }
    }
}

// The host threads the OpenMP loops may use.  A launcher may export OMP_NUM_THREADS=1 for its worker
// processes (torchrun does); the timed CPU baseline sets the count it wants explicitly.
void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
