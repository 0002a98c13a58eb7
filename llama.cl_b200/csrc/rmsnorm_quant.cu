// RMS normalization fused with the Q8 activation quantizer of the FCs that consume it.
//
// Replaces llmops.rmsnorm (ops/op_misc.hpp:142-181) followed by FC_dynamic_quantize_x (ops/op_fc.hpp:221-272)
// of every FC that reads the normalized activations: in the reference's decoder layer the output of
// input_layernorm feeds q_proj, k_proj and v_proj, the output of post_attention_layernorm feeds gate_proj and
// up_proj (chatllama/main.py:344-368), and each of those FCs quantizes the same values again.  Here the row is
// normalized and quantized once, into the pre-quantized activation format that q4fc_fc_decode_q8 reads
// (codes int8 [rows][Kg*G], then fp32 [Kg][16]: entry 2m = scale of row m, entry 2m+1 = its group sum).
//
// Bit-exactness.  The normalized values are bit-equal to the reference's:
//   * sum of squares: the reference keeps eight running sums, lane j adding x[8i+j]^2 for i = 0, 1, ... with
//     one fused multiply-add each, and folds them as ((s4+s0)+(s6+s2)) + ((s5+s1)+(s7+s3))
//     (ops/utils.hpp:92-98).  Eight lanes of one warp run exactly those eight chains (a dependent chain of
//     K/8 fma per lane, about a microsecond at K = 4096) out of shared memory, then the same fold.
//   * rms = sum / K, r = 1 / sqrt(rms + eps), y = (x * r) * w: IEEE division, square root and two separately
//     rounded multiplications, as the reference's scalar and AVX code do.
// The codes and scales then follow the quantizer's rules (quant_x.cu), so they are bit-equal to what the
// reference's FCs would compute from its own rmsnorm output; the group sums are tree-ordered like the decode
// kernel's.
//
// Optionally the residual addition in front of the normalization (llmops.iadd, chatllama/main.py:359) is done
// on the way in: the row that is normalized is x + residual (one IEEE add per element, as the reference's), and
// the sum can be written out as the new residual stream.
//
// One CTA per row: the row is first copied to shared memory by all warps, eight lanes run the chains, then
// every warp quantizes 128-k chunks (one 512-byte read of shared memory each).
#include <atomic>

#include "common.cuh"

namespace q4fc {
namespace {

constexpr int kRnThreads = 256;

__device__ __forceinline__ int sat8(int v) { return min(127, max(-128, v)); }

template <int G>
__global__ void __launch_bounds__(kRnThreads) rmsnorm_quant_kernel(const float* x, const float* residual,
                                                                   float* sum_out /* may alias x or residual */,
                                                                   int64_t K, int64_t ldx,
                                                                   const float* __restrict__ weight, float eps,
                                                                   float* __restrict__ y, int64_t ldy, int64_t Kg,
                                                                   int want_isum, int8_t* __restrict__ codes,
                                                                   float* __restrict__ sc) {
    extern __shared__ __align__(16) float row[];  // K floats, then one float for the factor
    constexpr int SEG = G / 4;
    constexpr int GPC = 128 / G;
    const int m = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* src = x + m * ldx;
    pdl_launch_dependents();
    pdl_wait_prior_grid();  // the activations may come from the kernel before

    for (int64_t i = threadIdx.x * 4; i < K; i += kRnThreads * 4) {  // K % 8 == 0 (checked by the launcher)
        float4 a = __ldcg(reinterpret_cast<const float4*>(src + i));
        if (residual != nullptr) {
            // the reference's iadd in front of the normalization (ops/op_misc.hpp:55-79): one IEEE add each
            const float4 b = __ldcg(reinterpret_cast<const float4*>(residual + m * ldx + i));
            a.x = __fadd_rn(a.x, b.x), a.y = __fadd_rn(a.y, b.y), a.z = __fadd_rn(a.z, b.z), a.w = __fadd_rn(a.w, b.w);
            if (sum_out != nullptr) *reinterpret_cast<float4*>(sum_out + m * ldx + i) = a;
        }
        *reinterpret_cast<float4*>(row + i) = a;
    }
    __syncthreads();

    if (warp == 0) {
        float s = 0.0f;
        if (lane < 8) {
            // the reference's lane `lane` of its 8-wide running sum
#pragma unroll 8
            for (int64_t i = lane; i < K; i += 8) s = __fmaf_rn(row[i], row[i], s);
        }
        // ((s4 + s0) + (s6 + s2)) + ((s5 + s1) + (s7 + s3))
        const float a = __fadd_rn(__shfl_sync(0xffffffffu, s, (lane & 3) + 4), __shfl_sync(0xffffffffu, s, lane & 3));
        const float b = __fadd_rn(a, __shfl_sync(0xffffffffu, a, (lane & 1) + 2));  // lanes 0, 1: a[j] + a[j+2]
        const float c = __fadd_rn(__shfl_sync(0xffffffffu, b, 0), __shfl_sync(0xffffffffu, b, 1));
        if (lane == 0) {
            const float rms = __fdiv_rn(c, (float)K);
            row[K] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(rms, eps)));
        }
    }
    __syncthreads();
    const float r = row[K];

    const int64_t chunks = (Kg * G + 127) / 128;
    for (int64_t c = warp; c < chunks; c += kRnThreads / 32) {
        const int64_t k = c * 128 + lane * 4;
        const int64_t kb = c * GPC + lane / SEG;
        const bool exists = kb < Kg;
        const int len = exists ? (int)min((int64_t)G, K - kb * G) : 0;
        const int body = len & ~7;
        const int e0 = (lane % SEG) * 4;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (k + 4 <= K) {
            const float4 a = *reinterpret_cast<const float4*>(row + k);
            const float4 w = __ldg(reinterpret_cast<const float4*>(weight + k));
            v[0] = __fmul_rn(__fmul_rn(a.x, r), w.x), v[1] = __fmul_rn(__fmul_rn(a.y, r), w.y);
            v[2] = __fmul_rn(__fmul_rn(a.z, r), w.z), v[3] = __fmul_rn(__fmul_rn(a.w, r), w.w);
            if (y != nullptr) *reinterpret_cast<float4*>(y + m * ldy + k) = make_float4(v[0], v[1], v[2], v[3]);
        }
        float amax = 0.0f, fsum = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (e0 + j < len) {
                amax = fmaxf(amax, fabsf(v[j]));
                fsum += v[j];
            }
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
}

}  // namespace

int launch_rmsnorm_quant(const float* x, const float* residual, float* sum_out, int rows, int64_t K, int64_t ldx,
                         const float* weight, float eps, float* y,
                         int64_t ldy, int G, bool want_isum, int8_t* codes, float* sc, bool pdl, cudaStream_t s) {
    if (rows == 0) return Q4FC_OK;
    const DeviceInfo* di = device_info();
    if (!di) return Q4FC_ECUDA;
    const int64_t Kg = (K + G - 1) / G;
    const size_t smem = (size_t)(K + 4) * sizeof(float);
    if (smem > (size_t)di->max_smem_optin) {
        set_error("rmsnorm_quant: a row of K=%lld floats does not fit the %d bytes of shared memory", (long long)K,
                  di->max_smem_optin);
        return Q4FC_ELIMIT;
    }
    const void* fn = (G == 32) ? reinterpret_cast<const void*>(&rmsnorm_quant_kernel<32>)
                               : reinterpret_cast<const void*>(&rmsnorm_quant_kernel<128>);
    static std::atomic<bool> attr_done[64][2] = {};  // set once per device; a second setter repeats the same call
    int dev = 0;
    Q4FC_CUDA_OK(cudaGetDevice(&dev));
    if (smem > 48 * 1024 && (dev >= 64 || !attr_done[dev][G == 128])) {
        Q4FC_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin));
        if (dev < 64) attr_done[dev][G == 128] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(kRnThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    int wi = want_isum ? 1 : 0;
    void* args[] = {&x,   &residual, &sum_out, &K,  &ldx,   &weight, &eps,
                    &y,   &ldy,      const_cast<int64_t*>(&Kg), &wi, &codes, &sc};
    Q4FC_CUDA_OK(cudaLaunchKernelExC(&cfg, fn, args));
    return Q4FC_OK;
}

}  // namespace q4fc
