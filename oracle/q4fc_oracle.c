/*
 * CPU ORACLE -- TEST INFRASTRUCTURE ONLY.
 *
 * Scalar, plain-C restatement of the quantized fully-connected path of
 * usstq/llama.cl (ops/op_fc.hpp, ops/utils.hpp).  It exists so that the CUDA
 * kernels can be checked on the same inputs; the shipped library never links,
 * loads or calls it.  Only tests/, the smoke check and the benchmark's
 * CPU-baseline leg may use it.
 *
 * Parity status: PINNED.  The restatement is compared bit-for-bit with the
 * reference's own code compiled from its sources (oracle/_ref, see
 * build_oracle.py), with golden vectors generated from that compiled reference
 * (tests/golden), and with the reference's own known-answer construction
 * (ops/test_ops.py:106-149: lossless Q4_1 packing, FC equal to fp32 linear).
 *
 * Block layout (ops/op_fc.hpp:14-24, 64-71), one block = 32 columns x G k:
 *   int8  w[G/8][128]   byte (k>>3)*128 + n*4 + (k&3); low nibble when
 *                       ((k>>2)&1)==0, else high nibble      (op_fc.hpp:39-48)
 *   fp16  wd[32]        scale per column
 *   fp16  wm[32]        minimum per column (Q4_1 only)
 * Packed tensor: [Ng][Kg][block bytes], C-contiguous.
 *
 * qtype: 0 = Q4_0 (symmetric, levels -7..7), 1 = Q4_1 (asymmetric, 0..15).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define Q4FC_GROUP_N 32

/* ---- fp16 <-> fp32, round-to-nearest-even (ops/utils.hpp:81-90: vcvtps2ph in
 * the current rounding mode, vcvtph2ps) ---------------------------------- */
static uint16_t f32_to_f16_rn(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? (0x0200u | ((absx >> 13) & 0x3FFu)) : 0u));
    }
    if (absx >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) { /* < 2^-25 (or == 2^-25 tie to even zero) */
        return (uint16_t)sign;
    }
    int32_t exp = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
    uint32_t shift;
    uint32_t hexp;
    if (exp < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - exp));
        hexp = 0;
    } else {
        shift = 13;
        hexp = (uint32_t)(exp + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    uint32_t h;
    if (hexp == 0) {
        h = q; /* may carry into the exponent field: that is the right value */
    } else {
        h = ((hexp - 1) << 10) + q; /* q holds the implicit bit: adds 1 to the exponent */
    }
    return (uint16_t)(sign | h);
}

static float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t x;
    if (exp == 0) {
        if (man == 0) {
            x = sign;
        } else {
            int e = -1;
            do {
                e++;
                man <<= 1;
            } while (!(man & 0x400u));
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        x = sign | 0x7F800000u | (man << 13);
    } else {
        x = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* exported for tests of the conversion itself */
uint16_t oracle_f32_to_f16(float f) { return f32_to_f16_rn(f); }
float oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

int oracle_block_bytes(int qtype, int G) {
    if ((qtype != 0 && qtype != 1) || G <= 0 || (G % 8)) return -1;
    return 16 * G + (qtype ? 128 : 64);
}

static inline uint8_t* nib_byte(uint8_t* blk, int k, int n) { return blk + (k >> 3) * 128 + n * 4 + (k & 3); }

static inline void nib_set(uint8_t* blk, int k, int n, int v) { /* op_fc.hpp:39-48 */
    uint8_t* p = nib_byte(blk, k, n);
    if ((k >> 2) & 1)
        *p = (uint8_t)((*p & 0x0F) | ((v & 0xF) << 4));
    else
        *p = (uint8_t)((*p & 0xF0) | (v & 0x0F));
}

static inline int nib_get_u(const uint8_t* blk, int k, int n) { /* op_fc.hpp:49-57: read UNSIGNED */
    const uint8_t* p = blk + (k >> 3) * 128 + n * 4 + (k & 3);
    return ((k >> 2) & 1) ? ((*p >> 4) & 0xF) : (*p & 0xF);
}

/* ---- weight packer: offline_FC_quant_Q4A, op_fc.hpp:151-219 --------------
 * w is [N][K] row-major fp32.  out is [Ng][Kg][BS].  Columns n >= N get
 * d = m = 0; the reference leaves their nibbles uninitialised, here they are
 * zero.  A ragged last K group (K % G != 0) scans only the valid elements
 * (the reference scans G elements past the row end there, which is not a
 * defined result); codes for k >= K are 0 as in op_fc.hpp:207-211. */
int oracle_pack(const float* w, int64_t N, int64_t K, int qtype, int G, uint8_t* out) {
    int BS = oracle_block_bytes(qtype, G);
    if (BS < 0 || N < 0 || K < 0) return 1;
    int64_t Ng = (N + Q4FC_GROUP_N - 1) / Q4FC_GROUP_N;
    int64_t Kg = (K + G - 1) / G;
#pragma omp parallel for schedule(static)
    for (int64_t nb = 0; nb < Ng; nb++) {
        for (int64_t kb = 0; kb < Kg; kb++) {
            uint8_t* blk = out + (nb * Kg + kb) * (int64_t)BS;
            memset(blk, 0, (size_t)BS);
            uint16_t* wd = (uint16_t*)(blk + 16 * G);
            uint16_t* wm = (uint16_t*)(blk + 16 * G + 64);
            int64_t k0 = kb * G;
            int len = (int)((K - k0) < G ? (K - k0) : G);
            for (int ni = 0; ni < Q4FC_GROUP_N; ni++) {
                int64_t n = nb * Q4FC_GROUP_N + ni;
                if (n >= N) continue; /* d = m = 0 already */
                const float* src = w + n * K + k0;
                /* get_min_max, op_fc.hpp:112-122: strict compares, first value wins ties */
                float vmin = src[0], vmax = src[0];
                for (int i = 1; i < len; i++) {
                    float a = src[i];
                    if (vmax < a) vmax = a;
                    if (vmin > a) vmin = a;
                }
                float d, m, id, lo, hi;
                if (qtype == 1) { /* op_fc.hpp:185-193 */
                    hi = 15.0f;
                    lo = 0.0f;
                    d = (vmax - vmin) / hi;
                    m = vmin;
                    id = (d != 0) ? (1.0f / d) : 0;
                    wd[ni] = f32_to_f16_rn(d);
                    wm[ni] = f32_to_f16_rn(m);
                } else { /* op_fc.hpp:194-203 */
                    hi = 7.0f;
                    lo = -7.0f;
                    float amax = fmaxf(fabsf(vmin), fabsf(vmax));
                    d = amax / hi;
                    m = 0.0f;
                    id = (d != 0) ? (1.0f / d) : 0;
                    wd[ni] = f32_to_f16_rn(d);
                }
                for (int ki = 0; ki < G; ki++) { /* op_fc.hpp:205-213 */
                    int q = 0;
                    if (ki < len) {
                        float r = roundf((src[ki] - m) * id); /* half away from zero */
                        float c = fminf(hi, fmaxf(r, lo));
                        q = (int)(int8_t)c;
                    }
                    nib_set(blk, ki, ni, q);
                }
            }
        }
    }
    return 0;
}

/* ---- offline_FC_dequant_Q4A, op_fc.hpp:124-149: out is [Ng*32][Kg*G].
 * The nibble is read unsigned for BOTH block types (op_fc.hpp:95-106), so a
 * Q4_0 tensor does not dequantize to the weights it was packed from.
 * nibble_signed != 0 selects the sign-corrected reading instead (not what the
 * reference computes; offered by the CUDA library as an option). */
int oracle_dequant(const uint8_t* wq, int64_t Ng, int64_t Kg, int qtype, int G, int nibble_signed, float* out) {
    int BS = oracle_block_bytes(qtype, G);
    if (BS < 0) return 1;
    int64_t ldo = Kg * G;
#pragma omp parallel for schedule(static)
    for (int64_t nb = 0; nb < Ng; nb++) {
        for (int64_t kb = 0; kb < Kg; kb++) {
            const uint8_t* blk = wq + (nb * Kg + kb) * (int64_t)BS;
            const uint16_t* wd = (const uint16_t*)(blk + 16 * G);
            const uint16_t* wm = (const uint16_t*)(blk + 16 * G + 64);
            for (int ni = 0; ni < Q4FC_GROUP_N; ni++) {
                float d = f16_to_f32(wd[ni]);
                float m = qtype ? f16_to_f32(wm[ni]) : 0.0f;
                for (int ki = 0; ki < G; ki++) {
                    int q = nib_get_u(blk, ki, ni);
                    if (nibble_signed && qtype == 0 && q >= 8) q -= 16;
                    float v = d * (float)q; /* exact: 11-bit x 4-bit */
                    out[(nb * 32 + ni) * ldo + kb * G + ki] = qtype ? (v + m) : v;
                }
            }
        }
    }
    return 0;
}

/* ---- FC_dynamic_quantize_x, op_fc.hpp:221-272 ---------------------------
 * x [rows][K] fp32 -> codes int8 [rows][Kg*G], scales fp32 [rows][Kg],
 * gsums fp32 [rows][Kg].  amax: utils.hpp:177-197.  Codes: utils.hpp:200-220
 * -- the 8-wide body rounds half to even (_mm256_round_ps NEAREST) and
 * saturates to int8 through packs; the scalar tail (len % 8 elements) uses
 * std::round (half away).  Group sum: sequential fp32 over the raw values. */
int oracle_quant_x(const float* x, int64_t rows, int64_t K, int G, float scale,
                   int8_t* codes, float* scales, float* gsums) {
    if (G <= 0 || rows < 0 || K < 0) return 1;
    int64_t Kg = (K + G - 1) / G;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t kb = 0; kb < Kg; kb++) {
            const float* src = x + r * K + kb * G;
            int8_t* q = codes + r * Kg * G + kb * G;
            int64_t left = K - kb * G;
            int len = (int)(left < G ? left : G);
            float amax = 0.0f;
            for (int i = 0; i < len; i++) {
                float a = fabsf(src[i]);
                if (amax < a) amax = a;
            }
            const float d = amax / 127;
            const float id = (d != 0) ? (1.0f / d) : 0;
            scales[r * Kg + kb] = d * scale;
            const int body = (len / 8) * 8; /* covered by the 8-wide loop */
            int i;
            for (i = 0; i < body; i++) {
                float v = rintf(src[i] * id); /* default rounding mode: nearest even */
                if (v > 127.0f) v = 127.0f;
                if (v < -128.0f) v = -128.0f;
                q[i] = (int8_t)v;
            }
            for (i = body; i < len; i++) q[i] = (int8_t)roundf(src[i] * id);
            for (i = len; i < G; i++) q[i] = 0;
            if (gsums) {
                float s = 0.0f;
                for (i = 0; i < len; i++) s += src[i];
                gsums[r * Kg + kb] = s;
            }
        }
    }
    return 0;
}

/* ---- fc_Q4A, op_fc.hpp:286-426 -----------------------------------------
 * y[r][n] for r < rows, n < N.  Per (row, column), groups in order:
 *   I   = sum_k nibble_u(n,k) * code(r,k)            exact int32
 *         (Q4_0: the nibble is pre-shifted by 4, still unsigned, and the
 *          activation scale carries the 1/16: op_fc.hpp:315,364-376)
 *   acc = fmaf(fp32(wd)*xs, (float)I, acc)           product rounded first
 *   acc = fmaf(fp32(wm), gsum, acc)                  Q4_1 only
 * The integer dot follows the dpbusd form of vnni() (utils.hpp:223-229): no
 * int16 saturation.  nibble_signed != 0 (Q4_0 only) sign-extends the nibble,
 * which is NOT what the reference computes.
 * Scratch: the activation quantization is done inside, as in the reference. */
int oracle_fc(const float* x, int64_t rows, int64_t K, const uint8_t* wq, int64_t Ng, int64_t Kg,
              int qtype, int G, int64_t N, int nibble_signed, float* y, int64_t ldy) {
    int BS = oracle_block_bytes(qtype, G);
    if (BS < 0 || rows < 0) return 1;
    if ((K + G - 1) / G != Kg) return 2;
    if (N > Ng * 32) return 3;
    int64_t Kp = Kg * G;
    int8_t* codes = (int8_t*)malloc((size_t)(rows * Kp + 64));
    float* xs = (float*)malloc((size_t)(rows * Kg + 1) * sizeof(float));
    float* gs = (float*)malloc((size_t)(rows * Kg + 1) * sizeof(float));
    if (!codes || !xs || !gs) {
        free(codes);
        free(xs);
        free(gs);
        return 4;
    }
    float scale = qtype ? 1.0f : (1.0f / 16.0f);
    oracle_quant_x(x, rows, K, G, scale, codes, xs, gs);
#pragma omp parallel for schedule(static)
    for (int64_t nb = 0; nb < Ng; nb++) {
        for (int64_t r = 0; r < rows; r++) {
            float acc[32];
            for (int ni = 0; ni < 32; ni++) acc[ni] = 0.0f;
            for (int64_t kb = 0; kb < Kg; kb++) {
                const uint8_t* blk = wq + (nb * Kg + kb) * (int64_t)BS;
                const uint16_t* wd = (const uint16_t*)(blk + 16 * G);
                const uint16_t* wm = (const uint16_t*)(blk + 16 * G + 64);
                const int8_t* q = codes + r * Kp + kb * G;
                float dx = xs[r * Kg + kb];
                float gsum = gs[r * Kg + kb];
                for (int ni = 0; ni < 32; ni++) {
                    int32_t I = 0;
                    for (int k8 = 0; k8 < G / 8; k8++) {
                        const uint8_t* wb = blk + k8 * 128 + ni * 4;
                        for (int j = 0; j < 4; j++) {
                            int lo = wb[j] & 0xF, hi = (wb[j] >> 4) & 0xF;
                            if (qtype == 0) {
                                if (nibble_signed) {
                                    if (lo >= 8) lo -= 16;
                                    if (hi >= 8) hi -= 16;
                                }
                                lo *= 16;
                                hi *= 16;
                            }
                            I += lo * (int32_t)q[k8 * 8 + j] + hi * (int32_t)q[k8 * 8 + 4 + j];
                        }
                    }
                    float d = f16_to_f32(wd[ni]) * dx;
                    acc[ni] = fmaf(d, (float)I, acc[ni]);
                    if (qtype) acc[ni] = fmaf(f16_to_f32(wm[ni]), gsum, acc[ni]);
                }
            }
            for (int ni = 0; ni < 32; ni++) {
                int64_t n = nb * 32 + ni;
                if (n < N) y[r * ldy + n] = acc[ni];
            }
        }
    }
    free(codes);
    free(xs);
    free(gs);
    return 0;
}

/* ---- rmsnorm, op_misc.hpp:142-181, in place on x [rows][K] ------------------
 * Eight running sums: lane j takes x[8i+j]^2 for i = 0, 1, ... with one fused
 * multiply-add each (vfmadd); they are folded as ((s4+s0)+(s6+s2)) +
 * ((s5+s1)+(s7+s3)) (_mm256_reduce_add_ps, utils.hpp:92-98).  rms = sum / K,
 * r = 1 / sqrt(rms + eps), x = (x * r) * w with both products rounded. */
int oracle_rmsnorm(float* x, int64_t rows, int64_t K, const float* w, float eps) {
    if (K % 8 != 0) return 1; /* the reference asserts hidden_states % 8 == 0 */
    for (int64_t m = 0; m < rows; m++) {
        float* src = x + m * K;
        float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int64_t i = 0; i < K; i += 8)
            for (int j = 0; j < 8; j++) s[j] = fmaf(src[i + j], src[i + j], s[j]);
        float a[4];
        for (int j = 0; j < 4; j++) a[j] = s[4 + j] + s[j];
        const float b0 = a[0] + a[2], b1 = a[1] + a[3];
        const float sum = b0 + b1;
        const float rms = sum / (float)K;
        const float r = 1.0f / sqrtf(rms + eps);
        for (int64_t i = 0; i < K; i++) {
            float v = src[i] * r;
            src[i] = v * w[i];
        }
    }
    return 0;
}

/* exp_ps_avx2 (ops/utils.hpp:293-371) for one value: clamp to [log(FLT_MIN), log(FLT_MAX)], n = floor(x*log2e + 0.5),
 * r = x - n*ln2 (one fused multiply-add), degree-5 polynomial in r (Horner, fused), times 2^(n-1), times 2;
 * inputs below log(FLT_MIN) give 0. */
static float ref_expf(float x) {
    union { uint32_t u; float f; } lo = {0xc2aeac50u}, hi = {0x42b17218u}, log2e = {0x3fb8aa3bu}, ln2 = {0x3f317218u},
        p1 = {0x3f7ffffbu}, p2 = {0x3efffee3u}, p3 = {0x3e2aad40u}, p4 = {0x3d2b9d0du}, p5 = {0x3c07cfceu}, two_n;
    const int zero = x < lo.f;
    if (x > hi.f) x = hi.f;
    if (x < lo.f) x = lo.f;
    float fx = floorf(x * log2e.f + 0.5f);
    const float r = fmaf(-fx, ln2.f, x);
    fx -= 1.0f;
    two_n.u = (uint32_t)((int32_t)lrintf(fx) + 127) << 23;
    float y = p5.f;
    y = fmaf(y, r, p4.f);
    y = fmaf(y, r, p3.f);
    y = fmaf(y, r, p2.f);
    y = fmaf(y, r, p1.f);
    y = fmaf(y, r, 1.0f);
    y = y * (zero ? 0.0f : two_n.f);
    return y * 2.0f;
}

/* llmops.itrans(gate, "silu") then llmops.imul(up, gate) (ops/op_misc.hpp:83-138, chatllama/main.py:365-368):
 * out = up * (gate * sigmoid(gate)), sigmoid(v) = rcp(1 + exp(-v)).  The reference's rcp is _mm256_rcp_ps, a
 * hardware approximation (relative error <= 1.5 * 2^-12) that plain C cannot reproduce bit for bit; this
 * restatement divides exactly, so it agrees with the compiled reference to about 4e-4 relative -- the golden
 * rows of tests/golden/silu_mul_ref.npz pin it to that. */
int oracle_silu_mul(const float* gate, const float* up, int64_t n, float* out) {
    for (int64_t i = 0; i < n; i++) {
        const float sig = 1.0f / (1.0f + ref_expf(0.0f - gate[i]));
        out[i] = up[i] * (gate[i] * sig);
    }
    return 0;
}

/* ---- per-channel int8 weights ("Q8C") of the older extension ----------------------------------------------
 * FC_quant_Q8C (ext/llama_ext.cpp:56-113): per output column n, amax over the whole row of W, d = amax / 127,
 * q = roundf(w / d) (half away from zero); blocks of 32 columns x 32 k, byte (k >> 2) * 128 + n * 4 + (k & 3)
 * (q8_c_block, ext/llama_ext.cpp:50-54); columns n >= N and k >= K are zero.  wq: int8 [Ng][Kg][1024],
 * scales: fp32 [Ng * 32]. */
int oracle_q8c_pack(const float* w, int64_t N, int64_t K, int8_t* wq, float* scales) {
    const int64_t Ng = (N + 31) / 32, Kg = (K + 31) / 32;
    memset(wq, 0, (size_t)(Ng * Kg * 1024));
    for (int64_t n = 0; n < Ng * 32; n++) {
        if (n >= N) {
            scales[n] = 0.0f;
            continue;
        }
        const float* src = w + n * K;
        float amax = 0.0f;
        for (int64_t k = 0; k < K; k++) {
            const float a = fabsf(src[k]);
            if (amax < a) amax = a;
        }
        const float d = amax / 127;
        const float id = (d != 0) ? (1.0f / d) : 0;
        scales[n] = d;
        int8_t* blk = wq + (n / 32) * Kg * 1024;
        const int noff = (int)(n % 32);
        for (int64_t k = 0; k < K; k++) {
            const int ki = (int)(k % 32);
            blk[(k / 32) * 1024 + (ki >> 2) * 128 + noff * 4 + (ki & 3)] = (int8_t)roundf(src[k] * id);
        }
    }
    return 0;
}

/* FC_evaluate_Q8C (ext/llama_ext.cpp:232-371): the activations are quantized per 32-group with scale 1 and no
 * group sums (FC_dynamic_quantize_x, :116-166); per (row, column) the groups in order:
 *   I = sum_k code(r,k) * q(n,k)  exact (the sign/maddubs form of :289-307 cannot saturate: |code| <= 127),
 *   acc = fmaf(dx[kb], (float)I, acc);   y = d_w[n] * acc  (:326-333). */
int oracle_q8c_fc(const float* x, int64_t rows, int64_t K, const int8_t* wq, const float* wscales, int64_t Ng,
                  int64_t Kg, int64_t N, float* y, int64_t ldy) {
    if ((K + 31) / 32 != Kg || N > Ng * 32) return 1;
    int8_t* codes = (int8_t*)malloc((size_t)(rows * Kg * 32 + 1));
    float* xs = (float*)malloc(sizeof(float) * (size_t)(rows * Kg + 1));
    if (!codes || !xs) return 2;
    oracle_quant_x(x, rows, K, 32, 1.0f, codes, xs, NULL);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        const int8_t* blk = wq + (n / 32) * Kg * 1024;
        const int noff = (int)(n % 32);
        for (int64_t r = 0; r < rows; r++) {
            float acc = 0.0f;
            for (int64_t kb = 0; kb < Kg; kb++) {
                int32_t I = 0;
                for (int ki = 0; ki < 32; ki++)
                    I += (int32_t)codes[r * Kg * 32 + kb * 32 + ki] *
                         (int32_t)blk[kb * 1024 + (ki >> 2) * 128 + noff * 4 + (ki & 3)];
                acc = fmaf(xs[r * Kg + kb], (float)I, acc);
            }
            y[r * ldy + n] = wscales[n] * acc;
        }
    }
    free(codes);
    free(xs);
    return 0;
}

/* embedding_q8c_quant_w (ops/op_embedding.hpp:51-78): per row of the table one scale d = amax / 127 and codes by
 * quant_row_q8_0 over the whole row (8-wide body half to even, scalar tail half away). */
int oracle_emb_q8c_quant(const float* w, int64_t V, int64_t E, int8_t* codes, float* scales) {
    for (int64_t b = 0; b < V; b++) {
        float s;
        if (oracle_quant_x(w + b * E, 1, E, (int)E, 1.0f, codes + b * E, &s, NULL)) return 1;
        scales[b] = s;
    }
    return 0;
}

/* embedding_q8c (ops/op_embedding.hpp:80-137): out[i][k] = scales[id] * (float)codes[id][k]. */
int oracle_emb_q8c(const int64_t* ids, int64_t n, const int8_t* codes, const float* scales, int64_t E, float* out) {
    for (int64_t i = 0; i < n; i++)
        for (int64_t k = 0; k < E; k++) out[i * E + k] = scales[ids[i]] * (float)codes[ids[i] * E + k];
    return 0;
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}
