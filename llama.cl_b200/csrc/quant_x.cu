// Stand-alone Q8 activation quantizer.
//
// Replaces FC_dynamic_quantize_x (ops/op_fc.hpp:221-272) with get_amax and
// quant_row_q8_0 (ops/utils.hpp:177-220): per row and K group
//   amax = max|x|, d = amax/127, id = 1/d (0 when d == 0),
//   scales = d * scale, codes = sat_s8(round(x * id)), gsums = sum of raw x.
// Rounding follows the reference exactly: the first floor(len/8)*8 elements
// of a group round half to even (its 8-wide AVX2 body), the remaining
// len % 8 elements round half away from zero (its scalar tail); padding codes
// are 0.  The group sum is accumulated sequentially in k order so that it is
// bit-equal to the reference's loop (ops/op_fc.hpp:262-268).
//
// One warp owns 128 consecutive k of one row: a 512-byte coalesced read, four
// values per lane.  The absolute maximum is a segmented butterfly over the
// G/4 lanes of a group.  The raw values are parked in shared memory so that
// one lane per group can walk them in order for the sequential sum; many
// resident warps hide that serial chain.  The decode FC kernel has its own
// fused copy of this arithmetic (tree-ordered sums); this kernel serves the
// prefill path and callers that want the quantized activations themselves.
#include "common.cuh"

namespace q4fc {
namespace {

constexpr int kQxWarps = 8;

__device__ __forceinline__ int sat8(int v) { return min(127, max(-128, v)); }

template <int G>
__global__ void __launch_bounds__(kQxWarps * 32) quant_x_kernel(const float* __restrict__ x, int64_t rows, int64_t K,
                                                                int64_t ldx, int64_t Kg, float scale, int vec_ok,
                                                                int8_t* __restrict__ codes, float* __restrict__ scales,
                                                                float* __restrict__ gsums) {
    constexpr int SEG = G / 4;     // lanes per group
    constexpr int GPC = 128 / G;   // groups per 128-k chunk
    constexpr int PADG = G + 1;    // padded group pitch in shared memory
    __shared__ float raw[kQxWarps][GPC * PADG + 3];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t chunks = (Kg * G + 127) / 128;
    const int64_t unit = (int64_t)blockIdx.x * kQxWarps + warp;
    if (unit >= rows * chunks) return;
    const int64_t row = unit / chunks;
    const int64_t c = unit % chunks;
    const int64_t k = c * 128 + lane * 4;
    const float* src = x + row * ldx + k;

    float v[4];
    if (vec_ok && k + 4 <= K) {
        float4 a = __ldg(reinterpret_cast<const float4*>(src));
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w;
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = (k + j < K) ? __ldg(src + j) : 0.0f;
    }

    const int g_l = lane / SEG;              // group inside the chunk
    const int64_t kb = c * GPC + g_l;        // group index in the row
    const bool group_exists = kb < Kg;
    const int len = group_exists ? (int)min((int64_t)G, K - kb * G) : 0;
    const int body = (len / 8) * 8;
    const int e0 = (lane % SEG) * 4;         // element index of v[0] inside the group

    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; j++)
        if (e0 + j < len) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
    for (int off = SEG / 2; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off, SEG));

    const float d = div_const_rn(amax, 127.0f, 1.0f / 127.0f);
    const float id = inv_or_zero(d);

    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int e = e0 + j;
        int q = 0;
        if (e < len) {
            const float t = __fmul_rn(v[j], id);
            if (e < body) {
                q = sat8(__float2int_rn(t));  // nearest even, as _mm256_round_ps + packs
            } else {
                const float h = __int_as_float((__float_as_int(t) & 0x80000000) | 0x3F000000);
                q = sat8(__float2int_rz(__fadd_rz(t, h)));  // std::round: half away
            }
        }
        packed |= (uint32_t)(q & 0xFF) << (8 * j);
    }
    if (group_exists) {
        *reinterpret_cast<uint32_t*>(codes + row * (Kg * G) + k) = packed;
        if (lane % SEG == 0) scales[row * Kg + kb] = __fmul_rn(d, scale);
    }

    if (gsums != nullptr) {
        float* mine = raw[warp];
#pragma unroll
        for (int j = 0; j < 4; j++) mine[g_l * PADG + e0 + j] = v[j];
        __syncwarp();
        if (lane < GPC) {
            const int64_t kb2 = c * GPC + lane;
            if (kb2 < Kg) {
                const int len2 = (int)min((int64_t)G, K - kb2 * G);
                float s = 0.0f;
                for (int i = 0; i < len2; i++) s = __fadd_rn(s, mine[lane * PADG + i]);
                gsums[row * Kg + kb2] = s;
            }
        }
    }
}

// Quantizer in front of the decode FC when rows x K is large.  The decode kernel normally quantizes the
// activations itself, every cluster for itself; beyond a few tens of thousands of values that repeated work
// costs more than one extra small launch.  One warp owns 128 consecutive k of ONE row, so the whole input is
// spread over hundreds of warps and the kernel is a single short latency chain.  Codes and scales follow
// the same rules as quant_x_kernel; the group sums are formed in exactly the order of the decode kernel's
// own quantizer (four values per lane in k order, then a butterfly over the group's lanes), so the FC
// result does not depend on which of the two quantized the input.
//   codes: int8 [rows][Kg*G];   sc: fp32 [Kg][16], entry 2*m = scale d of row m, entry 2*m + 1 = group sum
//   (or, for the signed-nibble Q4_0 form, the bits of the integer 8 * sum of codes).
//
// With `up` given the value that is quantized is silu(x) * up -- the MLP's gate activation and the product with
// the up projection (llmops.itrans(gate, "silu") then llmops.imul(up, gate), ops/op_misc.hpp:83-138,
// chatllama/main.py:365-368), i.e. the input of the down projection -- and `prod`, when given, receives those
// fp32 values.  silu(g) = g / (1 + exp(-g)) with expf and an IEEE division; the reference evaluates exp by a
// degree-5 polynomial and the reciprocal by _mm256_rcp_ps (relative error up to 3.7e-4), so the products agree
// with it to about 4e-4 relative, inside the 1e-3 / 1e-4 output tolerance, not bit for bit.
template <int G>
__device__ __forceinline__ void quant_pre_unit(const float* __restrict__ x, int rows, int64_t K, int64_t ldx, int64_t Kg,
                                               int vec_ok, int want_isum, int early_release, int8_t* __restrict__ codes,
                                               float* __restrict__ sc, const float* __restrict__ up,
                                               float* __restrict__ prod, int64_t ldp, int64_t unit) {
    constexpr int SEG = G / 4;
    constexpr int GPC = 128 / G;
    const int lane = threadIdx.x & 31;
    const int64_t chunks = (Kg * G + 127) / 128;
    // In a chain of programmatic launches the FC kernel behind this one should start as early as it can:
    // its start-up then runs beside the FC before.
    if (early_release) pdl_launch_dependents();
    if (unit >= chunks * rows) return;  // (an exited warp counts as having released the dependent launch)
    const int64_t c = unit / rows;
    const int m = (int)(unit - c * rows);
    const int64_t k = c * 128 + lane * 4;
    const int64_t kb = c * GPC + lane / SEG;
    const bool exists = kb < Kg;
    const int len = exists ? (int)min((int64_t)G, K - kb * G) : 0;
    const int body = len & ~7;
    const int e0 = (lane % SEG) * 4;
    pdl_wait_prior_grid();  // the activations may come from the kernel before

    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const float* src = x + m * ldx + k;
    if (vec_ok && k + 4 <= K) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(src));
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w;
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (k + j < K) v[j] = __ldcg(src + j);
    }
    if (up != nullptr) {
        float u[4] = {0.f, 0.f, 0.f, 0.f};
        const float* usrc = up + m * ldx + k;
        if (vec_ok && k + 4 <= K) {
            const float4 a = __ldcg(reinterpret_cast<const float4*>(usrc));
            u[0] = a.x, u[1] = a.y, u[2] = a.z, u[3] = a.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (k + j < K) u[j] = __ldcg(usrc + j);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float sg = __fdiv_rn(v[j], __fadd_rn(1.0f, expf(-v[j])));
            v[j] = __fmul_rn(u[j], sg);
        }
        if (prod != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (k + j < K) prod[m * ldp + k + j] = v[j];
        }
    }
    float amax = 0.0f, fsum = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; j++)
        if (e0 + j < len) {
            amax = fmaxf(amax, fabsf(v[j]));
            fsum += v[j];
        }
    // Otherwise the FC kernel behind this launch is released only now, with this warp's activations in
    // registers: its first act is to request megabytes of weights, and these few loads would queue behind
    // that stream.
    if (!early_release) pdl_launch_dependents();
#pragma unroll
    for (int off = SEG / 2; off > 0; off >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        fsum += __shfl_xor_sync(0xffffffffu, fsum, off);
    }
    const float d = div_const_rn(amax, 127.0f, 1.0f / 127.0f);
    const float id = inv_or_zero(d);
    uint32_t packed = 0;
    int isum = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        int q = 0;
        if (e0 + j < len) {
            const float t = __fmul_rn(v[j], id);
            if (e0 + j < body) {
                q = __float2int_rn(t);
            } else {
                const float h = __int_as_float((__float_as_int(t) & 0x80000000) | 0x3F000000);
                q = __float2int_rz(__fadd_rz(t, h));
            }
            q = sat8(q);
        }
        isum += q;
        packed |= (uint32_t)(q & 0xFF) << (8 * j);
    }
    if (want_isum) {
#pragma unroll
        for (int off = SEG / 2; off > 0; off >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, off);
    }
    if (exists) {
        *reinterpret_cast<uint32_t*>(codes + m * (Kg * G) + k) = packed;
        if (e0 == 0) {
            sc[kb * 16 + m * 2 + 0] = d;
            sc[kb * 16 + m * 2 + 1] = want_isum ? __int_as_float(8 * isum) : fsum;
        }
    }
}

template <int G>
__global__ void __launch_bounds__(128) quant_x_pre_kernel(const float* __restrict__ x, int rows, int64_t K,
                                                          int64_t ldx, int64_t Kg, int vec_ok, int want_isum,
                                                          int early_release, int8_t* __restrict__ codes,
                                                          float* __restrict__ sc, const float* __restrict__ up,
                                                          float* __restrict__ prod, int64_t ldp) {
    quant_pre_unit<G>(x, rows, K, ldx, Kg, vec_ok, want_isum, early_release, codes, sc, up, prod, ldp,
                      (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5));
}

// Several inputs in one launch (a batch of independent FCs has as many inputs to quantize, and each launch of its own
// would cost more than its work): the warps of the grid are dealt out to the inputs in order.
constexpr int kMaxQuantBatch = 16;
struct QuantBatch {
    const float* x[kMaxQuantBatch];
    int8_t* codes[kMaxQuantBatch];
    float* sc[kMaxQuantBatch];
    int64_t K[kMaxQuantBatch], ldx[kMaxQuantBatch];
    int rows[kMaxQuantBatch], vec_ok[kMaxQuantBatch];
    int unit0[kMaxQuantBatch + 1];  // first warp of input i; [n] = warps in all
    int n;
};
template <int G>
__global__ void __launch_bounds__(128) quant_x_pre_batch_kernel(const __grid_constant__ QuantBatch b, int want_isum,
                                                                int early_release) {
    const int unit = (int)blockIdx.x * 4 + (threadIdx.x >> 5);
    int i = 0;
    while (i + 1 < b.n && unit >= b.unit0[i + 1]) i++;
    const int64_t Kg = (b.K[i] + G - 1) / G;
    if (unit >= b.unit0[b.n]) {
        if (early_release) pdl_launch_dependents();
        return;
    }
    quant_pre_unit<G>(b.x[i], b.rows[i], b.K[i], b.ldx[i], Kg, b.vec_ok[i], want_isum, early_release, b.codes[i], b.sc[i],
                      nullptr, nullptr, 0, (int64_t)(unit - b.unit0[i]));
}

}  // namespace

int launch_quant_x_pre_batch(const q4fc_xq_call* calls, int n, int G, bool want_isum, bool pdl, cudaStream_t s) {
    QuantBatch b = {};
    int units = 0;
    for (int i = 0; i < n; i++) {
        const q4fc_xq_call& c = calls[i];
        if (c.rows == 0) continue;
        const int64_t Kg = (c.K + G - 1) / G;
        const int64_t chunks = (Kg * G + 127) / 128;
        uint8_t* base = static_cast<uint8_t*>(c.xq);
        const int k = b.n++;
        b.x[k] = c.x, b.rows[k] = (int)c.rows, b.K[k] = c.K, b.ldx[k] = c.ldx;
        b.codes[k] = reinterpret_cast<int8_t*>(base);
        b.sc[k] = reinterpret_cast<float*>(base + align_up((size_t)(c.rows * Kg * G), 256));
        b.vec_ok[k] = (c.K % 4 == 0) && (c.ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(c.x) & 15) == 0);
        b.unit0[k] = units;
        if (chunks * c.rows > 0x3fffffff - units) {
            set_error("quant_x_q8_batch: too many values for one launch");
            return Q4FC_ELIMIT;
        }
        units += (int)(chunks * c.rows);
    }
    if (b.n == 0) return Q4FC_OK;
    b.unit0[b.n] = units;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((units + 3) / 4));
    cfg.blockDim = dim3(128);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    if (G == 32)
        Q4FC_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_x_pre_batch_kernel<32>, b, (int)want_isum, (int)pdl));
    else
        Q4FC_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_x_pre_batch_kernel<128>, b, (int)want_isum, (int)pdl));
    return Q4FC_OK;
}

size_t quant_pre_bytes(int64_t rows, int64_t K, int G) {
    const int64_t Kg = (K + G - 1) / G;
    return align_up((size_t)(rows * Kg * G), 256) + align_up((size_t)Kg * 16 * sizeof(float), 256);
}

int launch_quant_x_pre(const float* x, int rows, int64_t K, int64_t ldx, int G, bool want_isum, int8_t* codes,
                       float* sc, bool pdl, cudaStream_t s, const float* up, float* prod, int64_t ldp) {
    const int64_t Kg = (K + G - 1) / G;
    const int64_t chunks = (Kg * G + 127) / 128;
    const int64_t grid = (chunks * rows + 3) / 4;
    const int vec_ok = (K % 4 == 0) && (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(up) & 15) == 0);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(128);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    if (G == 32)
        Q4FC_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_x_pre_kernel<32>, x, rows, K, ldx, Kg, vec_ok, (int)want_isum,
                                        (int)pdl, codes, sc, up, prod, ldp));
    else
        Q4FC_CUDA_OK(cudaLaunchKernelEx(&cfg, quant_x_pre_kernel<128>, x, rows, K, ldx, Kg, vec_ok, (int)want_isum,
                                        (int)pdl, codes, sc, up, prod, ldp));
    return Q4FC_OK;
}

int launch_quant_x(const float* x, int64_t rows, int64_t K, int64_t ldx, int G, float scale, int8_t* codes,
                   float* scales, float* gsums, cudaStream_t s) {
    const int64_t Kg = (K + G - 1) / G;
    if (rows == 0 || Kg == 0) return Q4FC_OK;
    const int64_t chunks = (Kg * G + 127) / 128;
    const int64_t grid = (rows * chunks + kQxWarps - 1) / kQxWarps;
    if (grid > 0x7fffffffLL) {
        set_error("quant_x: %lld x %lld exceeds the grid limit", (long long)rows, (long long)K);
        return Q4FC_ELIMIT;
    }
    const int vec_ok = (K % 4 == 0) && (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    if (G == 32)
        quant_x_kernel<32><<<(unsigned)grid, kQxWarps * 32, 0, s>>>(x, rows, K, ldx, Kg, scale, vec_ok, codes, scales,
                                                                    gsums);
    else
        quant_x_kernel<128><<<(unsigned)grid, kQxWarps * 32, 0, s>>>(x, rows, K, ldx, Kg, scale, vec_ok, codes,
                                                                     scales, gsums);
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

}  // namespace q4fc
