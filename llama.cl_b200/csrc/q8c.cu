// Per-channel int8 weights ("Q8C"): the FC of the reference's older extension and its quantized embedding table.
//
//   FC_quant_Q8C       ext/llama_ext.cpp:56-113    -> q8c_pack_kernel
//   FC_evaluate_Q8C    ext/llama_ext.cpp:232-371   -> quant_x_kernel<32> (scale 1, no group sums) + q8c_fc_kernel
//   embedding_q8c_quant_w   ops/op_embedding.hpp:51-78    -> emb_q8c_quant_kernel
//   embedding_q8c           ops/op_embedding.hpp:80-137   -> emb_q8c_kernel
//
// Weight layout (q8_c_block, ext/llama_ext.cpp:50-54): int8 [Ng][Kg][1024], one block = 32 columns x 32 k as 8 rows
// of 128 B; the 32-bit word n of row r holds k = 4r..4r+3 of column n.  fp32 scales [Ng*32], one per column:
// d = amax(row of W) / 127, q = roundf(w / d).
//
// FC arithmetic per (row m, column n), groups kb in order:  acc = fmaf(dx[m][kb], (float)I, acc) with
// I = sum over the group of code(m,k) * q(n,k) (exact), then y = d_w[n] * acc.  This kernel splits K over the warps
// of a CTA (and over the CTAs of a cluster when there are few stripes) and adds the partial sums in a fixed order,
// so a result differs from the reference's single chain by fp32 rounding only (and is the same from run to run).
//
// One mma.sync.m16n8k32.s8.s8 covers 16 columns x 32 k x 8 rows with the weight columns on the 16-row side: lane
// (g, t) loads 16 bytes of block row t and of block row 4 + t at byte 16 g -- the words of columns 4g..4g+3 -- so a
// warp reads a block as two coalesced 512-byte lines, and feeds columns 4g, 4g+1 to one MMA and 4g+2, 4g+3 to a
// second.  The activation codes and scales are read through L1 (every warp of every CTA reads the same few KB);
// the weights bypass it.
#include <cooperative_groups.h>

#include "common.cuh"
#include "decode_math.cuh"

namespace cg = cooperative_groups;

namespace q4fc {
namespace {

constexpr int kFcWarps = 8;
constexpr int kMaxSplit = 8;

__device__ __forceinline__ void mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float round_half_away(float t) {
    const float h = __int_as_float((__float_as_int(t) & 0x80000000) | 0x3F000000);
    return truncf(__fadd_rz(t, h));
}

// ---- pack ----------------------------------------------------------------------------------------------------------
// Two launches.  q8c_scale_kernel: one warp per column n (a row of W) finds amax and stores d = amax / 127.
// q8c_pack_kernel: grid (stripes, chunks of kPackBlocks K groups); per block the CTA reads 32 columns x 32 k with
// thread t on column t / 8, k = 4 (t % 8)..+3 -- eight threads read 128 contiguous bytes of a row of W -- turns its
// four values into one word, and the words cross shared memory so that the 1 KB block leaves as one coalesced line.
constexpr int kPackBlocks = 16;

__global__ void __launch_bounds__(256) q8c_scale_kernel(const float* __restrict__ w, int64_t N, int64_t K, int64_t n_pad,
                                                        int vec_ok, float* __restrict__ wscales) {
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= n_pad) return;
    float amax = 0.0f;
    if (n < N) {
        const float* src = w + n * K;
        if (vec_ok) {
            for (int64_t k = lane * 4; k < K; k += 128) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(src + k));
                amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
            }
        } else {
            for (int64_t k = lane; k < K; k += 32) amax = fmaxf(amax, fabsf(__ldg(src + k)));
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (lane == 0) wscales[n] = div_const_rn(amax, 127.0f, 1.0f / 127.0f);
}

__global__ void __launch_bounds__(256) q8c_pack_kernel(const float* __restrict__ w, int64_t N, int64_t K, int64_t Kg,
                                                       int vec_ok, const float* __restrict__ wscales,
                                                       int8_t* __restrict__ wq) {
    __shared__ uint32_t words[2][256];
    const int c = threadIdx.x >> 3, r = threadIdx.x & 7;
    const int64_t n = (int64_t)blockIdx.x * 32 + c;
    const float id = (n < N) ? inv_or_zero(wscales[n]) : 0.0f;
    const int64_t kb0 = (int64_t)blockIdx.y * kPackBlocks;
    const int64_t kb1 = min(Kg, kb0 + kPackBlocks);
    uint32_t* dst = reinterpret_cast<uint32_t*>(wq + ((int64_t)blockIdx.x * Kg + kb0) * 1024) + threadIdx.x;
    for (int64_t kb = kb0; kb < kb1; kb++, dst += 256) {
        uint32_t word = 0;
        if (n < N) {
            const int64_t k = kb * 32 + r * 4;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (vec_ok && k + 4 <= K) {
                const float4 a = __ldg(reinterpret_cast<const float4*>(w + n * K + k));
                v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (k + j < K) v[j] = __ldg(w + n * K + k + j);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int q = (int)round_half_away(__fmul_rn(v[j], id));  // 0 beyond K
                word |= (uint32_t)(q & 0xFF) << (8 * j);
            }
        }
        uint32_t* buf = words[(kb - kb0) & 1];
        buf[r * 32 + c] = word;
        __syncthreads();  // one barrier per block: the buffers alternate
        *dst = buf[threadIdx.x];
    }
}

// ---- FC ------------------------------------------------------------------------------------------------------------
// Grid (stripes * split, row tiles); a cluster of `split` CTAs shares one stripe and divides its K groups.  NT row
// tiles of 8 rows per CTA: the weights are loaded once per NT * 8 rows.
template <int NT>
__global__ void __launch_bounds__(kFcWarps * 32) q8c_fc_kernel(const int8_t* __restrict__ codes,
                                                               const float* __restrict__ xs, int64_t rows, int64_t Kg,
                                                               const int8_t* __restrict__ wq,
                                                               const float* __restrict__ wscales, int64_t N,
                                                               float* __restrict__ y, int64_t ldy, int split) {
    __shared__ float part[kFcWarps][NT][8][33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t stripe = blockIdx.x / split;
    const int rank = blockIdx.x % split;
    const int64_t row0 = (int64_t)blockIdx.y * (NT * 8);
    // K groups of this CTA: an even share, the first `rem` ranks one more
    const int64_t share = Kg / split, rem = Kg % split;
    const int64_t kb0 = rank * share + min((int64_t)rank, rem);
    const int64_t kb1 = kb0 + share + (rank < rem ? 1 : 0);

    float acc[NT][4][2];
#pragma unroll
    for (int i = 0; i < NT; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[i][c][0] = acc[i][c][1] = 0.0f;

    const int8_t* blk = wq + (stripe * Kg) * 1024 + t * 128 + g * 16;
    // rows whose codes (B fragment: row g of a tile) and scales (C fragment: rows 2t, 2t + 1) this lane reads
    const int8_t* crow[NT];
    const float* srow[NT][2];
    bool clive[NT], slive[NT][2];
#pragma unroll
    for (int i = 0; i < NT; i++) {
        const int64_t rb = row0 + i * 8;
        clive[i] = rb + g < rows;
        crow[i] = codes + (clive[i] ? rb + g : 0) * (Kg * 32) + 4 * t;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            slive[i][j] = rb + 2 * t + j < rows;
            srow[i][j] = xs + (slive[i][j] ? rb + 2 * t + j : 0) * Kg;
        }
    }

#pragma unroll 4
    for (int64_t kb = kb0 + warp; kb < kb1; kb += kFcWarps) {
        const uint4 lo = ldg_stream_v4(blk + kb * 1024);        // block row t: k = 4t..4t+3 of columns 4g..4g+3
        const uint4 hi = ldg_stream_v4(blk + kb * 1024 + 512);  // block row 4 + t: k = 16+4t..
#pragma unroll
        for (int i = 0; i < NT; i++) {
            uint32_t b0 = 0, b1 = 0;
            if (clive[i]) {
                b0 = __ldg(reinterpret_cast<const uint32_t*>(crow[i] + kb * 32));
                b1 = __ldg(reinterpret_cast<const uint32_t*>(crow[i] + kb * 32 + 16));
            }
            int c01[4] = {0, 0, 0, 0}, c23[4] = {0, 0, 0, 0};
            mma_s8s8(c01, lo.x, lo.y, hi.x, hi.y, b0, b1);  // columns 4g (c0, c1) and 4g + 1 (c2, c3)
            mma_s8s8(c23, lo.z, lo.w, hi.z, hi.w, b0, b1);  // columns 4g + 2 and 4g + 3
            const float d0 = slive[i][0] ? __ldg(srow[i][0] + kb) : 0.0f;
            const float d1 = slive[i][1] ? __ldg(srow[i][1] + kb) : 0.0f;
            acc[i][0][0] = fmaf(d0, (float)c01[0], acc[i][0][0]);
            acc[i][0][1] = fmaf(d1, (float)c01[1], acc[i][0][1]);
            acc[i][1][0] = fmaf(d0, (float)c01[2], acc[i][1][0]);
            acc[i][1][1] = fmaf(d1, (float)c01[3], acc[i][1][1]);
            acc[i][2][0] = fmaf(d0, (float)c23[0], acc[i][2][0]);
            acc[i][2][1] = fmaf(d1, (float)c23[1], acc[i][2][1]);
            acc[i][3][0] = fmaf(d0, (float)c23[2], acc[i][3][0]);
            acc[i][3][1] = fmaf(d1, (float)c23[3], acc[i][3][1]);
        }
    }
#pragma unroll
    for (int i = 0; i < NT; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) {
            part[warp][i][2 * t][4 * g + c] = acc[i][c][0];
            part[warp][i][2 * t + 1][4 * g + c] = acc[i][c][1];
        }
    __syncthreads();
    // warp 0's slot becomes the CTA's sum (warps in order)
    for (int e = threadIdx.x; e < NT * 8 * 32; e += kFcWarps * 32) {
        const int i = e / 256, m = (e / 32) % 8, c = e % 32;
        float s = part[0][i][m][c];
#pragma unroll
        for (int w2 = 1; w2 < kFcWarps; w2++) s += part[w2][i][m][c];
        part[0][i][m][c] = s;
    }
    if (split > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (rank == 0) {
            for (int e = threadIdx.x; e < NT * 8 * 32; e += kFcWarps * 32) {
                const int i = e / 256, m = (e / 32) % 8, c = e % 32;
                float s = part[0][i][m][c];
                for (int r = 1; r < split; r++) s += *cluster.map_shared_rank(&part[0][i][m][c], r);
                const int64_t row = row0 + i * 8 + m, n = stripe * 32 + c;
                if (row < rows && n < N) y[row * ldy + n] = __fmul_rn(__ldg(wscales + n), s);
            }
        }
        cluster.sync();  // the other CTAs' shared memory stays alive until rank 0 has read it
    } else {
        __syncthreads();
        for (int e = threadIdx.x; e < NT * 8 * 32; e += kFcWarps * 32) {
            const int i = e / 256, m = (e / 32) % 8, c = e % 32;
            const int64_t row = row0 + i * 8 + m, n = stripe * 32 + c;
            if (row < rows && n < N) y[row * ldy + n] = __fmul_rn(__ldg(wscales + n), part[0][i][m][c]);
        }
    }
}

// ---- embedding table -----------------------------------------------------------------------------------------------
// One CTA per table row: amax, then codes; the first floor(E / 8) * 8 values round half to even and the rest half
// away from zero, as quant_row_q8_0 (ops/utils.hpp:191-220) does over the whole row.
__global__ void __launch_bounds__(256) emb_q8c_quant_kernel(const float* __restrict__ table, int64_t E,
                                                            int8_t* __restrict__ codes, float* __restrict__ scales) {
    __shared__ float s_max[8];
    const float* src = table + (int64_t)blockIdx.x * E;
    int8_t* dst = codes + (int64_t)blockIdx.x * E;
    float amax = 0.0f;
    for (int64_t k = threadIdx.x; k < E; k += 256) amax = fmaxf(amax, fabsf(__ldg(src + k)));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = s_max[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = fmaxf(amax, s_max[i]);
    const float d = div_const_rn(amax, 127.0f, 1.0f / 127.0f);
    const float id = inv_or_zero(d);
    if (threadIdx.x == 0) scales[blockIdx.x] = d;
    const int64_t body = E & ~(int64_t)7;
    for (int64_t k = threadIdx.x; k < E; k += 256) {
        const float tv = __fmul_rn(__ldg(src + k), id);
        const int q = (k < body) ? __float2int_rn(tv) : (int)round_half_away(tv);
        dst[k] = (int8_t)min(127, max(-128, q));
    }
}

// One CTA per looked-up id: out[i][k] = scales[id] * (float)codes[id][k].  An id outside [0, V) leaves a row of
// zeros and sets bit 0x100 of the status word.
template <typename Tidx>
__global__ void __launch_bounds__(128) emb_q8c_kernel(const Tidx* __restrict__ ids, const int8_t* __restrict__ codes,
                                                      const float* __restrict__ scales, int64_t V, int64_t E,
                                                      float* __restrict__ out, int64_t ldo, int vec_ok,
                                                      int* __restrict__ status) {
    const int64_t i = blockIdx.x;
    const int64_t id = (int64_t)ids[i];
    float* dst = out + i * ldo;
    if (id < 0 || id >= V) {
        for (int64_t k = threadIdx.x; k < E; k += 128) dst[k] = 0.0f;
        if (threadIdx.x == 0 && status != nullptr) atomicOr(status, 0x100);
        return;
    }
    const int8_t* src = codes + id * E;
    const float s = __ldg(scales + id);
    if (vec_ok) {
        for (int64_t k = (int64_t)threadIdx.x * 16; k < E; k += 128 * 16) {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(src + k));
            const uint32_t wds[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float4 o;
                o.x = __fmul_rn(s, (float)(int8_t)(wds[j] & 0xFF));
                o.y = __fmul_rn(s, (float)(int8_t)((wds[j] >> 8) & 0xFF));
                o.z = __fmul_rn(s, (float)(int8_t)((wds[j] >> 16) & 0xFF));
                o.w = __fmul_rn(s, (float)(int8_t)(wds[j] >> 24));
                *reinterpret_cast<float4*>(dst + k + 4 * j) = o;
            }
        }
    } else {
        for (int64_t k = threadIdx.x; k < E; k += 128) dst[k] = __fmul_rn(s, (float)src[k]);
    }
}

}  // namespace

int launch_q8c_pack(const float* w, int64_t N, int64_t K, int8_t* wq, float* wscales, cudaStream_t s) {
    const int64_t Ng = (N + 31) / 32, Kg = (K + 31) / 32;
    if (Ng == 0) return Q4FC_OK;
    const int64_t chunks = (Kg + kPackBlocks - 1) / kPackBlocks;
    if (Ng > 0x7fffffffLL / 4 || chunks > 65535) {
        set_error("q8c_pack: %lld x %lld exceeds the grid limits", (long long)N, (long long)K);
        return Q4FC_ELIMIT;
    }
    const int vec_ok = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    q8c_scale_kernel<<<(unsigned)(Ng * 4), 256, 0, s>>>(w, N, K, Ng * 32, vec_ok, wscales);
    Q4FC_CUDA_OK(cudaGetLastError());
    if (Kg == 0) return Q4FC_OK;
    q8c_pack_kernel<<<dim3((unsigned)Ng, (unsigned)chunks), 256, 0, s>>>(w, N, K, Kg, vec_ok, wscales, wq);
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

size_t q8c_workspace_bytes(int64_t rows, int64_t K) {
    const int64_t Kg = (K + 31) / 32;
    return align_up((size_t)(rows * Kg * 32), 256) + align_up((size_t)(rows * Kg) * sizeof(float), 256);
}

int launch_q8c_fc(const float* x, int64_t rows, int64_t K, int64_t ldx, const int8_t* wq, const float* wscales,
                  int64_t Ng, int64_t Kg, int64_t N, float* y, int64_t ldy, void* ws, cudaStream_t s) {
    const DeviceInfo* di = device_info();
    if (!di) return Q4FC_ECUDA;
    int8_t* codes = static_cast<int8_t*>(ws);
    float* xs = reinterpret_cast<float*>(static_cast<char*>(ws) + align_up((size_t)(rows * Kg * 32), 256));
    if (int rc = launch_quant_x(x, rows, K, ldx, 32, 1.0f, codes, xs, nullptr, s)) return rc;
    const int64_t stripes = (N + 31) / 32;
    // few stripes: a cluster of CTAs shares each one, until the grid holds about two CTAs per SM
    int split = 1;
    while (split < kMaxSplit && stripes * split < 2 * (int64_t)di->sm_count && Kg / (2 * split) >= kFcWarps) split *= 2;
    const bool wide = rows > 8;
    const int64_t tiles = wide ? (rows + 31) / 32 : 1;
    if (stripes * split > 0x7fffffffLL || tiles > 65535) {
        set_error("q8c_fc: %lld rows x %lld columns exceed the grid limits", (long long)rows, (long long)N);
        return Q4FC_ELIMIT;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(stripes * split), (unsigned)tiles);
    cfg.blockDim = dim3(kFcWarps * 32);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int8_t* ccodes = codes;
    const float* cxs = xs;
    if (wide)
        Q4FC_CUDA_OK(cudaLaunchKernelEx(&cfg, q8c_fc_kernel<4>, ccodes, cxs, rows, Kg, wq, wscales, N, y, ldy, split));
    else
        Q4FC_CUDA_OK(cudaLaunchKernelEx(&cfg, q8c_fc_kernel<1>, ccodes, cxs, rows, Kg, wq, wscales, N, y, ldy, split));
    (void)Ng;
    return Q4FC_OK;
}

int launch_emb_q8c_quant(const float* table, int64_t V, int64_t E, int8_t* codes, float* scales, cudaStream_t s) {
    if (V == 0) return Q4FC_OK;
    if (V > 0x7fffffffLL) {
        set_error("emb_q8c_quant: %lld rows exceed the grid limit", (long long)V);
        return Q4FC_ELIMIT;
    }
    emb_q8c_quant_kernel<<<(unsigned)V, 256, 0, s>>>(table, E, codes, scales);
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

int launch_emb_q8c(const void* ids, int ids_are_i32, int64_t n, const int8_t* codes, const float* scales, int64_t V,
                   int64_t E, float* out, int64_t ldo, cudaStream_t s) {
    if (n == 0 || E == 0) return Q4FC_OK;
    if (n > 0x7fffffffLL) {
        set_error("emb_q8c: %lld ids exceed the grid limit", (long long)n);
        return Q4FC_ELIMIT;
    }
    const int vec_ok = (E % 16 == 0) && (ldo % 4 == 0) && ((reinterpret_cast<uintptr_t>(codes) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    int* status = ring_status_word();
    if (ids_are_i32)
        emb_q8c_kernel<int32_t><<<(unsigned)n, 128, 0, s>>>(static_cast<const int32_t*>(ids), codes, scales, V, E, out,
                                                            ldo, vec_ok, status);
    else
        emb_q8c_kernel<int64_t><<<(unsigned)n, 128, 0, s>>>(static_cast<const int64_t*>(ids), codes, scales, V, E, out,
                                                            ldo, vec_ok, status);
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

}  // namespace q4fc
