// Weight packer and dequantizer for the Q4_0 / Q4_1 block format.
//
// pack_kernel replaces offline_FC_quant_Q4A (ops/op_fc.hpp:151-219): fp32
// W[N][K] -> int8 [Ng][Kg][BS].  HBM-bound streaming kernel: 4 bytes read and
// 0.52-0.63 bytes written per weight.
//
// Work split: one thread owns one 32-bit output word = one column n x 8
// consecutive k (two 128-bit loads).  The G/8 threads that share a (column,
// K group) sit in adjacent lanes, so the group minimum / maximum is a
// segmented warp-shuffle reduction.  The reduction keeps the reference's
// "first value wins a tie" rule of get_min_max (ops/op_fc.hpp:112-122) by
// always combining an earlier k range (left) with a later one (right) under
// the same strict compares, which matters only for the sign of a zero
// minimum.  A CTA stages a tile of 32 columns x 256 k of packed output in
// shared memory and writes it out with 128-bit stores.
//
// Arithmetic is the reference's, in fp32 with IEEE division: Q4_1
// d=(max-min)/15, m=min, q=clamp(roundf((w-m)/d'),0,15) with d'=1/d computed
// first; Q4_0 d=max(|min|,|max|)/7, q=clamp(roundf(w*d'),-7,7).  roundf
// (half away from zero) is done as trunc(v +- 0.5) with the addition rounded
// toward zero, which is exact for every fp32 v.
#include "common.cuh"

namespace q4fc {
namespace {

constexpr int kPackThreads = 256;
constexpr int kTileK = 256;  // k covered by one CTA tile

struct MinMax {
    float vmin, vmax;
    int has;
};

__device__ __forceinline__ void mm_take(MinMax& a, float v) {  // sequential step of get_min_max
    if (a.vmax < v) a.vmax = v;
    if (a.vmin > v) a.vmin = v;
}

__device__ __forceinline__ int round_half_away(float v) {
    // trunc(v + copysign(0.5, v)) with a round-toward-zero add == roundf(v)
    float h = __int_as_float((__float_as_int(v) & 0x80000000) | 0x3F000000);
    return __float2int_rz(__fadd_rz(v, h));
}

template <int G, int QTYPE>
__global__ void __launch_bounds__(kPackThreads) pack_kernel(const float* __restrict__ w, int64_t N, int64_t K,
                                                            int64_t Kg, int tiles_k, int vec_ok,
                                                            uint8_t* __restrict__ out) {
    constexpr int BS = block_bytes(QTYPE, G);
    constexpr int SEG = G / 8;              // lanes sharing one (column, group)
    constexpr int NPW = 32 / SEG;           // columns per warp step
    constexpr int GB = kTileK / G;          // groups per CTA tile
    constexpr int UNITS = GB * (32 / NPW);  // warp steps per tile
    constexpr int ITERS = UNITS / (kPackThreads / 32);
    static_assert(UNITS % (kPackThreads / 32) == 0, "tile must divide among the warps");

    __shared__ __align__(16) uint32_t stage[GB * BS / 4];

    const int64_t nb = blockIdx.x / tiles_k;
    const int tile = blockIdx.x % tiles_k;
    const int64_t kb0 = (int64_t)tile * GB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg_lane = lane % SEG;  // = k8 inside the group

    float v[ITERS][8];
    int nvalid[ITERS];  // valid elements of this thread's 8 (prefix), -1: column beyond N

#pragma unroll
    for (int it = 0; it < ITERS; it++) {
        const int u = warp + it * (kPackThreads / 32);
        const int kb_l = u / (32 / NPW);
        const int n_l = (u % (32 / NPW)) * NPW + lane / SEG;
        const int64_t n = nb * 32 + n_l;
        const int64_t k = (kb0 + kb_l) * G + seg_lane * 8;
        int cnt = -1;
        if (n < N && kb0 + kb_l < Kg) {
            cnt = (int)min((int64_t)8, max((int64_t)0, K - k));
            const float* src = w + n * K + k;
            if (cnt == 8 && vec_ok) {
                float4 a = __ldg(reinterpret_cast<const float4*>(src));
                float4 b = __ldg(reinterpret_cast<const float4*>(src) + 1);
                v[it][0] = a.x, v[it][1] = a.y, v[it][2] = a.z, v[it][3] = a.w;
                v[it][4] = b.x, v[it][5] = b.y, v[it][6] = b.z, v[it][7] = b.w;
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) v[it][j] = (j < cnt) ? __ldg(src + j) : 0.0f;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) v[it][j] = 0.0f;
        }
        nvalid[it] = cnt;
    }

#pragma unroll
    for (int it = 0; it < ITERS; it++) {
        const int u = warp + it * (kPackThreads / 32);
        const int kb_l = u / (32 / NPW);
        const int n_l = (u % (32 / NPW)) * NPW + lane / SEG;
        const int cnt = nvalid[it];

        // Fast path (whole warp has 8 valid values per lane): plain min / max and an xor butterfly.
        // The value of a minimum / maximum does not depend on the scan order; only the SIGN of a zero
        // does (get_min_max keeps the first of equal values), so when any lane of the warp ends up with
        // a zero minimum or maximum, or values are missing, the warp redoes the reduction in order.
        float vmin = v[it][0], vmax = v[it][0];
#pragma unroll
        for (int j = 1; j < 8; j++) vmin = fminf(vmin, v[it][j]), vmax = fmaxf(vmax, v[it][j]);
#pragma unroll
        for (int off = 1; off < SEG; off <<= 1) {
            vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, off));
            vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
        }
        if (__any_sync(0xffffffffu, cnt != 8 || vmin == 0.0f || vmax == 0.0f)) {
            MinMax mm;
            mm.has = cnt > 0;
            mm.vmin = mm.vmax = v[it][0];
#pragma unroll
            for (int j = 1; j < 8; j++)
                if (j < cnt) mm_take(mm, v[it][j]);
            // ordered segmented reduction: lane i absorbs lane i+off (later k)
#pragma unroll
            for (int off = 1; off < SEG; off <<= 1) {
                float rmin = __shfl_down_sync(0xffffffffu, mm.vmin, off, SEG);
                float rmax = __shfl_down_sync(0xffffffffu, mm.vmax, off, SEG);
                int rhas = __shfl_down_sync(0xffffffffu, mm.has, off, SEG);
                if (seg_lane + off < SEG && rhas) {
                    if (mm.vmax < rmax) mm.vmax = rmax;
                    if (mm.vmin > rmin) mm.vmin = rmin;
                }
            }
            vmin = __shfl_sync(0xffffffffu, mm.vmin, 0, SEG);
            vmax = __shfl_sync(0xffffffffu, mm.vmax, 0, SEG);
        }

        float d, m, id;
        if (QTYPE == 1) {
            d = div_const_rn(__fsub_rn(vmax, vmin), 15.0f, 1.0f / 15.0f);
            m = vmin;
        } else {
            d = div_const_rn(fmaxf(fabsf(vmin), fabsf(vmax)), 7.0f, 1.0f / 7.0f);
            m = 0.0f;
        }
        id = inv_or_zero(d);

        uint32_t word = 0;
        if (cnt >= 0) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (j < cnt) {
                    // byte (j&3), low nibble for j<4, high nibble for j>=4 (ops/op_fc.hpp:39-48)
                    const uint32_t place = 1u << (8 * (j & 3) + 4 * (j >> 2));
                    if (QTYPE == 1) {
                        // (w - m) * id >= 0: roundf is trunc(t + 0.5) with the add rounded toward zero; clamp at 15
                        const float t = __fmul_rn(__fsub_rn(v[it][j], m), id);
                        const uint32_t q = (uint32_t)min(15, __float2int_rz(__fadd_rz(t, 0.5f)));
                        word += q * place;  // nibbles do not overlap: a multiply-add places the code
                    } else {
                        const int q = min(7, max(round_half_away(__fmul_rn(v[it][j], id)), -7));
                        word += (uint32_t)(q & 0xF) * place;
                    }
                }
            }
        }
        stage[kb_l * (BS / 4) + seg_lane * 32 + n_l] = word;
        if (seg_lane == 0) {
            uint16_t* tail = reinterpret_cast<uint16_t*>(stage + kb_l * (BS / 4) + G * 4);
            const bool live = cnt >= 0;  // cnt==0 cannot occur at seg_lane 0 of an existing group
            tail[n_l] = live ? f2h_rn(d) : (uint16_t)0;
            if (QTYPE == 1) tail[32 + n_l] = live ? f2h_rn(m) : (uint16_t)0;
        }
    }
    __syncthreads();

    const int groups_here = (int)min((int64_t)GB, Kg - kb0);
    const int n16 = groups_here * BS / 16;
    uint4* dst = reinterpret_cast<uint4*>(out + (nb * Kg + kb0) * (int64_t)BS);
    const uint4* src4 = reinterpret_cast<const uint4*>(stage);
    for (int i = threadIdx.x; i < n16; i += kPackThreads) dst[i] = src4[i];
}

template <int G, int QTYPE>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ wq, int64_t nblocks, int64_t Kg,
                                                      int nibble_signed, float* __restrict__ out) {
    // one thread per 32-bit word: column n, 8 consecutive k (ops/op_fc.hpp:124-149, get() :49-61 / :95-106)
    constexpr int BS = block_bytes(QTYPE, G);
    constexpr int WPB = G * 4;  // words per block
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= nblocks * WPB) return;
    const int64_t blk = gid / WPB;
    const int wi = (int)(gid % WPB);
    const int k8 = wi / 32, n = wi % 32;
    const uint8_t* b = wq + blk * BS;
    const uint32_t word = *reinterpret_cast<const uint32_t*>(b + k8 * 128 + n * 4);
    const float d = h2f(*reinterpret_cast<const uint16_t*>(b + 16 * G + 2 * n));
    const float m = QTYPE ? h2f(*reinterpret_cast<const uint16_t*>(b + 16 * G + 64 + 2 * n)) : 0.0f;
    const int64_t nb = blk / Kg, kb = blk % Kg;
    float* dst = out + (nb * 32 + n) * (Kg * G) + kb * G + k8 * 8;
    float r[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        int q = (word >> (8 * (j & 3) + 4 * (j >> 2))) & 0xF;
        if (QTYPE == 0 && nibble_signed && q >= 8) q -= 16;
        const float p = __fmul_rn(d, (float)q);  // exact: 11-bit x 4-bit
        r[j] = QTYPE ? __fadd_rn(p, m) : p;
    }
    reinterpret_cast<float4*>(dst)[0] = make_float4(r[0], r[1], r[2], r[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(r[4], r[5], r[6], r[7]);
}

}  // namespace

int launch_pack(const float* w, int64_t N, int64_t K, int qtype, int G, uint8_t* wq, cudaStream_t s) {
    const int64_t Ng = (N + 31) / 32, Kg = (K + G - 1) / G;
    if (Ng == 0 || Kg == 0) return Q4FC_OK;
    const int GB = kTileK / G;
    const int64_t tiles_k = (Kg + GB - 1) / GB;
    if (Ng * tiles_k > 0x7fffffffLL || tiles_k > 0x7fffffffLL) {
        set_error("pack: %lld x %lld tiles exceed the grid limit", (long long)Ng, (long long)tiles_k);
        return Q4FC_ELIMIT;
    }
    const int vec_ok = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    dim3 grid((unsigned)(Ng * tiles_k));
#define Q4FC_PACK(GG, QQ) \
    pack_kernel<GG, QQ><<<grid, kPackThreads, 0, s>>>(w, N, K, Kg, (int)tiles_k, vec_ok, wq)
    if (G == 32 && qtype == 1) Q4FC_PACK(32, 1);
    else if (G == 128 && qtype == 1) Q4FC_PACK(128, 1);
    else if (G == 32 && qtype == 0) Q4FC_PACK(32, 0);
    else Q4FC_PACK(128, 0);
#undef Q4FC_PACK
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

int launch_dequant(const uint8_t* wq, int64_t Ng, int64_t Kg, int qtype, int G, int nibble_signed, float* out,
                   cudaStream_t s) {
    const int64_t nblocks = Ng * Kg;
    if (nblocks == 0) return Q4FC_OK;
    const int64_t threads = nblocks * G * 4;
    const int64_t grid = (threads + 255) / 256;
    if (grid > 0x7fffffffLL) {
        set_error("dequant: tensor too large for one launch");
        return Q4FC_ELIMIT;
    }
#define Q4FC_DEQ(GG, QQ) dequant_kernel<GG, QQ><<<(unsigned)grid, 256, 0, s>>>(wq, nblocks, Kg, nibble_signed, out)
    if (G == 32 && qtype == 1) Q4FC_DEQ(32, 1);
    else if (G == 128 && qtype == 1) Q4FC_DEQ(128, 1);
    else if (G == 32 && qtype == 0) Q4FC_DEQ(32, 0);
    else Q4FC_DEQ(128, 0);
#undef Q4FC_DEQ
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

}  // namespace q4fc
