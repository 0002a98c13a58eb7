// Decode FC (rows <= 8): weight-streaming GEMV over the reference's packed
// Q4_0 / Q4_1 tensor.  Replaces fc_Q4A (ops/op_fc.hpp:286-426) for small
// B*M.  HBM-bound: every packed byte is read exactly once.
//
// Decomposition.  The packed tensor [Ng][Kg][BS] is one contiguous byte
// stream; its Ng*Kg blocks are dealt out in memory order, an equal contiguous
// run per CTA and, inside the CTA, an equal contiguous run per warp
// ("stream-K": every SM streams the same number of bytes whatever N and K
// are).  A run crosses stripe (32-column) boundaries freely; a warp keeps
// fp32 accumulators for the stripe it is in and emits a "segment" when the
// stripe changes.
//
// Inner product.  One lane loads 128 bits = 4 columns x 8 k of packed
// nibbles straight from global memory (a warp covers 512 contiguous bytes, 4
// block rows); `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F` are the two u8x4
// operands for k..k+3 and k+4..k+7 (ops/op_fc.hpp:39-48).  They feed
// mma.sync.m16n8k32 (u8 x s8 -> s32) with the 16-row side holding weight
// columns and the 8-column side holding the activation rows, so the group dot
// product is exact in int32 and costs the same for 1..8 rows.  The k order
// inside the MMA is permuted consistently on both operands.  Loads for the
// next step are issued before the current step is consumed; the registers
// are the staging buffer (~70 KB in flight per SM).
//
// Scaling (ops/op_fc.hpp:381-412) after every K group:
//   acc = fmaf(fp32(wd) * xs, (float)I, acc);  Q4_1: acc = fmaf(fp32(wm), gsum, acc)
// Q4_0 follows the reference's reading of the stored nibble as UNSIGNED
// (ops/op_fc.hpp:364-376); its x16 operand shift and 1/16 scale cancel exactly
// and are not materialised.  The SIGNED instantiation sign-extends instead:
// sum((nib ^ 8) * code) - 8 * sum(code).
//
// Activations.  Each CTA quantizes the rows itself (amax, codes, scale, group
// sum: ops/op_fc.hpp:246-268 with the rounding rules of ops/utils.hpp:200-220)
// into shared memory; codes and scales are bit-equal to the reference's, group
// sums are tree-ordered.  Under programmatic dependent launch the first
// weight loads are issued before the wait on the preceding kernel, since
// weights never depend on it.
//
// Reduction.  Warp segments that do not cover a whole stripe are summed per
// CTA in shared memory in warp order; stripes shared between CTAs go through
// a workspace slot per CTA plus an arrival counter per stripe, and the last
// CTA to arrive adds the slots in CTA order.  There is no spin-wait anywhere
// and the result does not depend on timing.
#include <atomic>

#include "common.cuh"
#include "decode_math.cuh"

namespace q4fc {
namespace {

constexpr int kDecWarps = 8;
constexpr int kDecThreads = kDecWarps * 32;

struct DecodeParams {
    const float* x;
    float* y;
    const uint8_t* wq;
    int* counters;
    float* partials;
    int64_t K, ldx, N, ldy;
    int rows;
    int Ng, Kg;
    int T;            // Ng * Kg
    int code_stride;  // bytes between code rows in shared memory
    int x_vec_ok, y_vec_ok;
};

// CTA that owns block b under the split start(c) = floor(c*T/P)
__device__ __forceinline__ int cta_of_block(int64_t b, int64_t T, int64_t P) { return (int)(((b + 1) * P + T - 1) / T - 1); }

template <int G, int QTYPE, bool SIGNED>
struct Dec {
    static constexpr int BS = block_bytes(QTYPE, G);
    static constexpr int SETS = G / 32;               // 4-row sets per block
    static constexpr int NBLK = (G == 32) ? 4 : 1;    // blocks per pipeline step

    struct Step {
        uint4 q[NBLK][SETS];
        uint2 wd[NBLK];
        uint2 wm[NBLK];
    };

    // lane (g,t): rows 4j+t of each set, 16-byte chunk g of the 128-byte row
    static __device__ __forceinline__ void load_step(Step& s, const uint8_t* wq, int b, int b_end, int g, int t) {
#pragma unroll
        for (int i = 0; i < NBLK; i++) {
            if (b + i < b_end) {
                const uint8_t* blk = wq + (int64_t)(b + i) * BS;
#pragma unroll
                for (int j = 0; j < SETS; j++) s.q[i][j] = ldg_stream_v4(blk + (4 * j + t) * 128 + g * 16);
                s.wd[i] = ldg_stream_v2(blk + 16 * G + g * 8);
                if (QTYPE == 1) s.wm[i] = ldg_stream_v2(blk + 16 * G + 64 + g * 8);
            }
        }
    }
};

template <int G, int QTYPE, bool SIGNED>
__global__ void __launch_bounds__(kDecThreads, 2) fc_decode_kernel(const DecodeParams p) {
    using D = Dec<G, QTYPE, SIGNED>;
    constexpr int BS = D::BS;
    constexpr int SETS = D::SETS;
    constexpr int NBLK = D::NBLK;

    extern __shared__ __align__(16) uint8_t smem[];
    // layout: wpart [W][2][8][32] f32 | seg_nb [W][2] int | sc [Kg][8][2] f32 | codes [rows][code_stride]
    float* wpart = reinterpret_cast<float*>(smem);
    int* seg_nb = reinterpret_cast<int*>(smem + kDecWarps * 2 * 8 * 32 * 4);
    float* sc = reinterpret_cast<float*>(smem + kDecWarps * 2 * 8 * 32 * 4 + 64);
    uint8_t* codes = reinterpret_cast<uint8_t*>(sc + (int64_t)p.Kg * 16);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t T = p.T, P = gridDim.x;
    const int cb0 = (int)(((int64_t)blockIdx.x * T) / P);
    const int cb1 = (int)(((int64_t)(blockIdx.x + 1) * T) / P);
    const int Lc = cb1 - cb0;
    const int wb0 = cb0 + (int)(((int64_t)warp * Lc) / kDecWarps);
    const int wb1 = cb0 + (int)(((int64_t)(warp + 1) * Lc) / kDecWarps);

    pdl_launch_dependents();

    // weights do not depend on the preceding kernel: start streaming them now
    typename D::Step cur, nxt;
    D::load_step(cur, p.wq, wb0, wb1, g, t);

    if (lane < 2) seg_nb[warp * 2 + lane] = -1;

    pdl_wait_prior_grid();

    // ---- quantize the activation rows into shared memory -------------------
    {
        constexpr int SEG = G / 4;    // lanes per group
        constexpr int GPC = 128 / G;  // groups per 128-k chunk
        const int64_t Kp = (int64_t)p.Kg * G;
        const int chunks = (int)((Kp + 127) / 128);
        for (int u = warp; u < p.rows * chunks; u += kDecWarps) {
            const int row = u / chunks, c = u % chunks;
            const int64_t k = (int64_t)c * 128 + lane * 4;
            const float* src = p.x + row * p.ldx + k;
            float v[1][4];
            if (p.x_vec_ok && k + 4 <= p.K) {
                float4 a = __ldcg(reinterpret_cast<const float4*>(src));
                v[0][0] = a.x, v[0][1] = a.y, v[0][2] = a.z, v[0][3] = a.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) v[0][j] = (k + j < p.K) ? __ldcg(src + j) : 0.0f;
            }
            const int kb = c * GPC + lane / SEG;
            const bool exists = kb < p.Kg;
            const int len = exists ? (int)min((int64_t)G, p.K - (int64_t)kb * G) : 0;
            uint32_t pk[1];
            float dq[1], aux[1];
            q8_quantize_rows<G, 1, SIGNED>(v, lane, len, pk, dq, aux);  // the arithmetic every decode kernel shares
            const uint32_t packed = pk[0];
            if (exists) {
                *reinterpret_cast<uint32_t*>(codes + (int64_t)row * p.code_stride + k) = packed;
                if (lane % SEG == 0) {
                    // reference: x_scales = d * scale with scale = 1/16 for Q4_0, cancelled by its
                    // x16 nibble shift; both are exact powers of two and are left out here
                    sc[kb * 16 + row * 2 + 0] = dq[0];
                    sc[kb * 16 + row * 2 + 1] = aux[0];
                }
            }
        }
    }
    __syncthreads();

    // ---- stream this warp's run of blocks ------------------------------------
    float acc[4][2];
#pragma unroll
    for (int i = 0; i < 4; i++) acc[i][0] = acc[i][1] = 0.0f;
    int nslot = 0;
    int b = wb0;
    int nb = (wb0 < wb1) ? wb0 / p.Kg : 0;
    int kb = (wb0 < wb1) ? wb0 % p.Kg : 0;
    int seg_kb0 = kb;
    const uint8_t* my_codes = codes + (int64_t)g * p.code_stride + 8 * t;
    const bool row_live = g < p.rows;

    auto emit = [&](int stripe, int kfirst, int kend) {
        const int64_t n0 = (int64_t)stripe * 32 + g * 4;
        if (kfirst == 0 && kend == p.Kg) {
#pragma unroll
            for (int mi = 0; mi < 2; mi++) {
                const int m = 2 * t + mi;
                if (m < p.rows) {
                    float* dst = p.y + m * p.ldy + n0;
                    if (p.y_vec_ok && n0 + 4 <= p.N) {
                        *reinterpret_cast<float4*>(dst) = make_float4(acc[0][mi], acc[1][mi], acc[2][mi], acc[3][mi]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            if (n0 + i < p.N) dst[i] = acc[i][mi];
                    }
                }
            }
        } else {
            float* slot = wpart + (warp * 2 + nslot) * 256;
#pragma unroll
            for (int mi = 0; mi < 2; mi++)
                *reinterpret_cast<float4*>(slot + (2 * t + mi) * 32 + g * 4) =
                    make_float4(acc[0][mi], acc[1][mi], acc[2][mi], acc[3][mi]);
            if (lane == 0) seg_nb[warp * 2 + nslot] = stripe;
            nslot++;
        }
#pragma unroll
        for (int i = 0; i < 4; i++) acc[i][0] = acc[i][1] = 0.0f;
    };

    auto process = [&](const typename D::Step& st) {
    #pragma unroll
        for (int i = 0; i < NBLK; i++) {
            if (b + i < wb1) {
                // the block arithmetic every decode kernel shares (exact integer sums, then the fp32 scaling)
                block_accumulate<G, QTYPE, SIGNED>(st.q[i], st.wd[i], st.wm[i], my_codes + (int64_t)kb * G, row_live,
                                                   sc + kb * 16, t, acc);
                // advance; close the segment at a stripe boundary
                kb++;
                if (kb == p.Kg) {
                    emit(nb, seg_kb0, kb);
                    kb = 0;
                    seg_kb0 = 0;
                    nb++;
                }
            }
        }
    };

    // two register sets take turns as the staging buffer for the loads in flight
    while (b < wb1) {
        D::load_step(nxt, p.wq, b + NBLK, wb1, g, t);
        process(cur);
        b += NBLK;
        if (b >= wb1) break;
        D::load_step(cur, p.wq, b + NBLK, wb1, g, t);
        process(nxt);
        b += NBLK;
    }
    if (kb != seg_kb0) emit(nb, seg_kb0, kb);  // run ended inside a stripe
    __syncthreads();

    // ---- combine warp segments per stripe, then across CTAs ------------------
    if (Lc <= 0) return;
    const int nbF = cb0 / p.Kg, nbL = (cb1 - 1) / p.Kg;
    for (int s = nbF + warp; s <= nbL; s += kDecWarps) {
        float sum[kMaxDecodeRows];
#pragma unroll
        for (int m = 0; m < kMaxDecodeRows; m++) sum[m] = 0.0f;
        bool found = false;
        for (int i = 0; i < kDecWarps * 2; i++) {
            if (seg_nb[i] == s) {
                found = true;
#pragma unroll
                for (int m = 0; m < kMaxDecodeRows; m++)
                    if (m < p.rows) sum[m] += wpart[i * 256 + m * 32 + lane];
            }
        }
        if (!found) continue;  // every segment of this stripe was complete and already stored
        const int64_t n = (int64_t)s * 32 + lane;
        const bool whole = ((int64_t)s * p.Kg >= cb0) && ((int64_t)(s + 1) * p.Kg <= cb1);
        if (whole) {
#pragma unroll
            for (int m = 0; m < kMaxDecodeRows; m++)
                if (m < p.rows && n < p.N) p.y[m * p.ldy + n] = sum[m];
            continue;
        }
        const int which = (s == nbF) ? 0 : 1;
        float* slot = p.partials + ((int64_t)blockIdx.x * 2 + which) * 256;
#pragma unroll
        for (int m = 0; m < kMaxDecodeRows; m++)
            if (m < p.rows) __stcg(slot + m * 32 + lane, sum[m]);
        __threadfence();
        __syncwarp();
        const int cF = cta_of_block((int64_t)s * p.Kg, T, P);
        const int cL = cta_of_block((int64_t)(s + 1) * p.Kg - 1, T, P);
        int last = 0;
        if (lane == 0) last = (atomicAdd(p.counters + s, 1) + 1 == cL - cF + 1);
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) continue;
        __threadfence();
#pragma unroll
        for (int m = 0; m < kMaxDecodeRows; m++) sum[m] = 0.0f;
        for (int c = cF; c <= cL; c++) {
            const int c_first_stripe = (int)((((int64_t)c * T) / P) / p.Kg);
            const float* src = p.partials + ((int64_t)c * 2 + (c_first_stripe == s ? 0 : 1)) * 256;
#pragma unroll
            for (int m = 0; m < kMaxDecodeRows; m++)
                if (m < p.rows) sum[m] += __ldcg(src + m * 32 + lane);
        }
#pragma unroll
        for (int m = 0; m < kMaxDecodeRows; m++)
            if (m < p.rows && n < p.N) p.y[m * p.ldy + n] = sum[m];
        if (lane == 0) p.counters[s] = 0;  // ready for the next call
    }
}

struct KernelEntry {
    const void* fn;
    bool attr_done[16];
};

template <int G, int QTYPE, bool SIGNED>
int launch_variant(const DecodeParams& p, size_t smem, int grid, unsigned flags, cudaStream_t s) {
    static std::atomic<bool> attr_done[64] = {};  // set once per device; a second setter repeats the same call
    int dev = 0;
    Q4FC_CUDA_OK(cudaGetDevice(&dev));
    auto* fn = fc_decode_kernel<G, QTYPE, SIGNED>;
    if (dev < 64 && !attr_done[dev]) {
        const DeviceInfo* di = device_info();
        if (!di) return Q4FC_ECUDA;
        Q4FC_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin));
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    int nattr = 0;
    if (flags & Q4FC_FLAG_PDL) {
        attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[nattr].val.programmaticStreamSerializationAllowed = 1;
        nattr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    Q4FC_CUDA_OK(cudaLaunchKernelEx(&cfg, fn, p));
    return Q4FC_OK;
}

constexpr int kCtasPerSm = 2;

}  // namespace

// Workspace layout (the same for every call, so that one workspace serves calls of any N):
//   [0, 256) status | CTA partials [ctas][2][8][32] fp32 | stripe counters int[Ng] ... up to 64 KB |
//   scratch of the quantizing launch in front of the cluster kernel (quant_x.cu), at a fixed offset so that
//   it never lands on counters of a call with another N
static size_t partials_bytes() {
    const DeviceInfo* di = device_info();
    const int sms = di ? di->sm_count : 256;
    return (size_t)sms * kCtasPerSm * 2 * 256 * sizeof(float);
}

size_t decode_prequant_offset() { return kWsStatusBytes + partials_bytes() + kWsCounterCapacity; }

size_t decode_workspace_bytes(int64_t N) {
    const int64_t Ng = (N + 31) / 32;
    return kWsStatusBytes + partials_bytes() + align_up((size_t)Ng * 4, 256);
}

int launch_fc_decode(const float* x, int rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng, int64_t Kg,
                     int qtype, int G, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes, unsigned flags,
                     cudaStream_t s) {
    if (rows == 0 || N == 0) return Q4FC_OK;
    const DeviceInfo* di = device_info();
    if (!di) return Q4FC_ECUDA;
    if (Ng * Kg >= 0x7fffffffLL) {
        set_error("fc_decode: %lld blocks exceed the 2^31 limit", (long long)(Ng * Kg));
        return Q4FC_ELIMIT;
    }
    if ((size_t)Ng * 4 > kWsCounterCapacity) {
        set_error("fc_decode: the stream-K kernel takes N <= %lld; use the default decode kernel",
                  (long long)(kWsCounterCapacity / 4 * 32));
        return Q4FC_ELIMIT;
    }
    // the kernel keeps a counter per stripe of the packed tensor, also of stripes beyond N
    if (ws == nullptr || ws_bytes < decode_workspace_bytes(Ng * 32)) {
        set_error("fc_decode: workspace of %zu bytes given, %zu needed", ws_bytes, decode_workspace_bytes(Ng * 32));
        return Q4FC_EWORKSPACE;
    }
    DecodeParams p;
    p.x = x, p.y = y, p.wq = wq;
    p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + kWsStatusBytes);
    p.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(ws) + kWsStatusBytes + partials_bytes());
    p.K = K, p.ldx = ldx, p.N = N, p.ldy = ldy;
    p.rows = rows, p.Ng = (int)Ng, p.Kg = (int)Kg, p.T = (int)(Ng * Kg);
    const int64_t Kp = Kg * G;
    // code rows 32 bytes apart modulo 128 keep the 8-byte operand loads of a half warp on distinct banks
    int64_t stride = (Kp + 127) / 128 * 128 + 32;
    p.code_stride = (int)stride;
    p.x_vec_ok = (K % 4 == 0) && (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    p.y_vec_ok = (ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
    const size_t smem = (size_t)kDecWarps * 2 * 8 * 32 * 4 + 64 + (size_t)Kg * 64 + (size_t)rows * stride;
    if (smem > (size_t)di->max_smem_optin) {
        set_error("fc_decode: rows=%d K=%lld needs %zu bytes of shared memory (limit %d)", rows, (long long)K, smem,
                  di->max_smem_optin);
        return Q4FC_ELIMIT;
    }
    int grid = di->sm_count * kCtasPerSm;
    if (grid > p.T) grid = p.T;
    const bool sgn = (flags & Q4FC_FLAG_NIBBLE_SIGNED) && qtype == 0;
    if (qtype == 1 && G == 32) return launch_variant<32, 1, false>(p, smem, grid, flags, s);
    if (qtype == 1 && G == 128) return launch_variant<128, 1, false>(p, smem, grid, flags, s);
    if (qtype == 0 && G == 32 && !sgn) return launch_variant<32, 0, false>(p, smem, grid, flags, s);
    if (qtype == 0 && G == 128 && !sgn) return launch_variant<128, 0, false>(p, smem, grid, flags, s);
    if (qtype == 0 && G == 32) return launch_variant<32, 0, true>(p, smem, grid, flags, s);
    return launch_variant<128, 0, true>(p, smem, grid, flags, s);
}

}  // namespace q4fc

// ---------------------------------------------------------------------------
// Decode FC for callers that cannot allocate device memory.
//
// Some hosts of this library hand every byte of device memory to their own
// arena when the process starts (serving runtimes that size their KV cache
// from "whatever is free"), or run under a memory budget in which a late
// cudaMalloc can fail or stall the device while it synchronizes.  Such a
// caller has nowhere to get the FC workspace from.  For it the partial sums
// and arrival counters of the stream-K reduction live in a fixed array that
// is part of the loaded library image: every GPU that loads the library
// holds kStaticScratchBytes (about 1.3 MB) until the process exits.
//
// The array is shared by every call on a device and keeps what the last call
// left in it.  The counters and the status word are cleared on the stream
// before each launch.  Two calls that may overlap on the GPU (different
// streams without an ordering between them) race on the array; order them.
//
// The first call on a device looks up the array's device address; make that
// first call outside any stream capture.
#include <mutex>

namespace q4fc {
namespace {
constexpr int kStaticMaxCtas = 640;        // room for 320 SMs at two CTAs each
constexpr int64_t kStaticMaxN = 262144;    // 8192 stripes of 32 columns
constexpr size_t kStaticScratchBytes =
    kWsStatusBytes + (size_t)kStaticMaxCtas * 2 * 256 * sizeof(float) + (size_t)(kStaticMaxN / 32) * sizeof(int);
}  // namespace
}  // namespace q4fc

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_static_scratch[q4fc::kStaticScratchBytes];

extern "C" __attribute__((visibility("default"))) int q4fc_fc_decode_noalloc(
    const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg, int qtype,
    int group_k, int64_t N, float* y, int64_t ldy, unsigned flags, q4fc_stream_t stream) {
    using namespace q4fc;
    static std::mutex mu;
    static void* dev_ptr[64] = {};
    if (!valid_variant(qtype, group_k)) {
        set_error("fc_decode_noalloc: unsupported block type (qtype=%d, group_k=%d)", qtype, group_k);
        return Q4FC_EVARIANT;
    }
    if (rows > kMaxDecodeRows) {
        set_error("fc_decode_noalloc: rows=%lld exceeds the %d rows the entry point takes", (long long)rows,
                  kMaxDecodeRows);
        return Q4FC_ELIMIT;
    }
    if (rows < 0 || K <= 0 || N < 0 || Kg <= 0 || (K + group_k - 1) / group_k != Kg || N > Ng * 32 || ldx < K ||
        ldy < N || (rows > 0 && N > 0 && (!x || !wq || !y))) {
        set_error("fc_decode_noalloc: bad sizes or null pointer (rows=%lld, K=%lld, Kg=%lld, N=%lld, Ng=%lld)",
                  (long long)rows, (long long)K, (long long)Kg, (long long)N, (long long)Ng);
        return Q4FC_EINVAL;
    }
    if ((reinterpret_cast<uintptr_t>(wq) & 15) || (reinterpret_cast<uintptr_t>(x) & 3) ||
        (reinterpret_cast<uintptr_t>(y) & 3)) {
        set_error("fc_decode_noalloc: packed weights need 16-byte alignment, x and y 4-byte");
        return Q4FC_EALIGN;
    }
    // the kernel keeps a counter per stripe of the packed tensor: the limit is on Ng, not only on N
    if (N > kStaticMaxN || Ng > kStaticMaxN / 32) {
        set_error("fc_decode_noalloc: N=%lld (Ng=%lld) exceeds the built-in scratch (N <= %lld); use q4fc_fc_decode "
                  "with a caller-provided workspace", (long long)N, (long long)Ng, (long long)kStaticMaxN);
        return Q4FC_ELIMIT;
    }
    if (rows == 0 || N == 0) return Q4FC_OK;
    const size_t need = decode_workspace_bytes(Ng * 32);
    if (need > kStaticScratchBytes) {
        set_error("fc_decode_noalloc: this GPU needs %zu bytes of scratch, the built-in array holds %zu", need,
                  (size_t)kStaticScratchBytes);
        return Q4FC_ELIMIT;
    }
    int dev = 0;
    Q4FC_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("fc_decode_noalloc: device index %d not supported", dev);
        return Q4FC_ELIMIT;
    }
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev_ptr[dev] == nullptr) {
            // set-up, once per device, with that device current
            void* p = nullptr;
            Q4FC_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
            dev_ptr[dev] = p;
        }
        scratch = dev_ptr[dev];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // what must start at zero: the status word and this call's stripe counters
    Q4FC_CUDA_OK(cudaMemsetAsync(scratch, 0, kWsStatusBytes, s));
    Q4FC_CUDA_OK(cudaMemsetAsync(static_cast<unsigned char*>(scratch) + need - align_up((size_t)Ng * 4, 256), 0,
                                 align_up((size_t)Ng * 4, 256), s));
    return launch_fc_decode(x, (int)rows, K, ldx, static_cast<const uint8_t*>(wq), Ng, Kg, qtype, group_k, N, y, ldy,
                            scratch, kStaticScratchBytes, flags, s);
}
