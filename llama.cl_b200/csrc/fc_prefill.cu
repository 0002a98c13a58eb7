// Prefill FC (rows > 8): dense int8 contraction on the 5th-generation tensor
// cores.  Replaces fc_Q4A (ops/op_fc.hpp:286-426) for large B*M.
//
//   y[m][n] = sum_kb  fp32(wd[n,kb]) * xs[m,kb] * I[m,n,kb]  (+ fp32(wm[n,kb]) * gsum[m,kb], Q4_1)
//   I[m,n,kb] = sum_{k in group kb} nibble(n,k) * code(m,k)      exact int32
//
// Two launches: the Q8 quantizer (quant_x.cu) writes codes / scales / group
// sums of all rows to the workspace, then this kernel runs the GEMM.
//
// One CTA computes a 128 (columns n) x 128 (rows m) output tile.
//   * operand A = weights: the packed nibbles of 4 stripes are unpacked to
//     one byte per weight in shared memory, K-major rows of 128 bytes, in the
//     128-byte-swizzle canonical layout that tcgen05.mma reads;
//   * operand B = activation codes (int8), same layout;
//   * D = int32 accumulators in tensor memory, lane = weight column,
//     column = activation row.
// Every K group has its own pair of scales, so a group's MMA(s) (one K=32
// instruction for group 32, four for group 128) write a fresh TMEM buffer
// (4 buffers x 128 columns = all 512 columns) and the epilogue warps read the
// buffer back with tcgen05.ld, turn the exact integers into fp32 (magic-number
// add, no cvt), scale them and accumulate the tile in registers.  The CUDA-core
// work per (m, n, group) -- one int add, one fp add, one mul, one or two fma --
// is what bounds this kernel: the tensor pipe waits for the epilogue.
//
// Warp roles (13 warps): 0-7 epilogue (warp%4 = TMEM lane quarter, warp/4 =
// half of the 128 tile rows), 8-11 producers (unpack A, copy B and the scales
// of one 128-k stage; generic-proxy stores + fence.proxy.async), 12 MMA issue
// (one elected lane).  mbarriers: full/empty per shared-memory stage,
// tfull/tempty per TMEM buffer.  Every wait is bounded: when a wait runs out
// the CTA sets the workspace status word, every role leaves its loop, TMEM is
// freed and the kernel returns.
#include "common.cuh"

namespace q4fc {
namespace {

constexpr int kTileN = 128;            // weight columns per tile = TMEM lanes
constexpr int kTileM = 128;            // activation rows per tile = TMEM columns per buffer
constexpr int kStageK = 128;           // k per shared-memory stage (one 128-byte swizzle row)
constexpr int kStages = 4;
constexpr int kTmemBufs = 4;
constexpr int kEpiWarps = 8, kProdWarps = 4;
constexpr int kProdThreads = kProdWarps * 32;
constexpr int kThreads = (kEpiWarps + kProdWarps + 1) * 32;
constexpr int kMmaWarp = kEpiWarps + kProdWarps;
constexpr uint64_t kWaitLimitNs = 1000000000ull;  // every mbarrier wait gives up after one second

// stage layout in shared memory (bytes); A and B tiles are 1024-byte aligned (swizzle atom)
constexpr int kABytes = kTileN * kStageK;          // 16 KB
constexpr int kBBytes = kTileM * kStageK;          // 16 KB
constexpr int kWscBytes = 4 * kTileN * 8;          // [group in stage][n] {wd, wm} fp32
constexpr int kXscBytes = 4 * kTileM * 8;          // [group in stage][m] {xs, gsum} fp32
constexpr int kStageBytes = kABytes + kBBytes + kWscBytes + kXscBytes;  // 40 KB
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct PrefillParams {
    const uint8_t* wq;
    const int8_t* codes;   // [rows][Kp]
    const float* xs;       // [rows][Kg]
    const float* gs;       // [rows][Kg]
    float* y;
    int* status;
    int64_t rows, N, ldy, Kp;
    int Ng, Kg;
};

// ---- PTX helpers -------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(1000u) /* suspend-time hint, ns */
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// bounded wait: gives up after kWaitLimitNs, or as soon as another role has raised the abort flag
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    for (uint32_t i = 1;; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 31) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > kWaitLimitNs) break;
        }
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile with 128-byte rows and 128-byte swizzle: rows 128 B apart, 8-row groups
// 1024 B apart (stride byte offset), descriptor version 1, layout type 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
// byte address of (row, byte-in-row) inside a swizzled tile
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t byte) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((((byte >> 4) ^ (row & 7)) & 7) << 4) + (byte & 15);
}

template <int G, int QTYPE, bool SIGNED>
__global__ void __launch_bounds__(kThreads, 1) fc_prefill_kernel(const PrefillParams p) {
    constexpr int BS = block_bytes(QTYPE, G);
    constexpr int GPS = kStageK / G;  // K groups per stage: 4 (group 32) or 1 (group 128)
    constexpr int MMAS = G / 32;      // K=32 instructions per group

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* bars = smem + kStages * kStageBytes;
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * kStages;
    const uint32_t bar_tfull = bar_empty + 8 * kStages, bar_tempty = bar_tfull + 8 * kTmemBufs;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8 * (2 * kStages + 2 * kTmemBufs));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tile = blockIdx.x, m_tile = blockIdx.y;
    const int64_t n0 = (int64_t)n_tile * kTileN, m0 = (int64_t)m_tile * kTileM;
    const int nb0 = n_tile * 4;
    const int nstage = (p.Kg + GPS - 1) / GPS;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; i++) {
            mbar_init(bar_full + 8 * i, kProdThreads);
            mbar_init(bar_empty + 8 * i, 1 + kEpiWarps);
        }
        for (int i = 0; i < kTmemBufs; i++) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, kEpiWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {  // one warp allocates all 512 TMEM columns (this kernel runs one CTA per SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= kEpiWarps && warp < kMmaWarp) {
        // =================== producers: one 128-k stage at a time ===================
        const int pt = threadIdx.x - kEpiWarps * 32;  // 0..127
        const int pw = pt >> 5;                       // stripe of the tile handled by this warp
        const int c = lane & 7, rr = lane >> 3;       // 16-byte chunk (columns 4c..4c+3), row inside a 4-row set
        const int nb = nb0 + pw;
        const bool stripe_live = nb < p.Ng;
        for (int it = 0; it < nstage; it++) {
            const int s = it % kStages;
            if (!mbar_wait(bar_empty + 8 * s, ((it / kStages) & 1) ^ 1, abort_flag)) break;
            uint8_t* st = smem + s * kStageBytes;
            const uint32_t a_base = smem_u32(st), b_base = a_base + kABytes;
            float2* wsc = reinterpret_cast<float2*>(st + kABytes + kBBytes);
            float2* xsc = reinterpret_cast<float2*>(st + kABytes + kBBytes + kWscBytes);
            const int kb0 = it * GPS;
            // ---- A: unpack nibbles of stripe nb: 16 word-rows (8 k each) x 32 columns
#pragma unroll
            for (int i4 = 0; i4 < 4; i4++) {
                const int r = 4 * i4 + rr;  // word-row inside the stage: k = 8r .. 8r+7
                uint4 w = make_uint4(0u, 0u, 0u, 0u);
                const int kb = (G == 128) ? kb0 : kb0 + (r >> 2);
                if (stripe_live && kb < p.Kg) {
                    const int row_in_block = (G == 128) ? r : (r & 3);
                    w = ldg_stream_v4(p.wq + ((int64_t)nb * p.Kg + kb) * BS + row_in_block * 128 + c * 16);
                }
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int col = (i + (c >> 1)) & 3;  // rotated order: a half warp covers all 8 swizzle rows
                    uint32_t lo = ww[col] & 0x0F0F0F0Fu, hi = (ww[col] >> 4) & 0x0F0F0F0Fu;
                    if (SIGNED) {  // sign-extend each nibble into its byte
                        lo |= (lo & 0x08080808u) * 0x1Eu;
                        hi |= (hi & 0x08080808u) * 0x1Eu;
                    }
                    const uint32_t row = pw * 32 + 4 * c + col;
                    const uint32_t addr = a_base + swz(row, 8 * r);
                    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(lo), "r"(hi) : "memory");
                }
            }
            // ---- B: codes of row m0 + pt, 128 bytes
            {
                const int64_t m = m0 + pt;
                const int8_t* src = p.codes + m * p.Kp + (int64_t)it * kStageK;
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (m < p.rows && (int64_t)it * kStageK + q * 16 < p.Kp) v = __ldg(reinterpret_cast<const uint4*>(src) + q);
                    const uint32_t addr = b_base + swz(pt, 16 * q);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
                                 "r"(v.w)
                                 : "memory");
                }
            }
            // ---- scales of the stage's groups
#pragma unroll
            for (int gi = 0; gi < GPS; gi++) {
                const int kb = kb0 + gi;
                float2 wv = make_float2(0.f, 0.f), xv = make_float2(0.f, 0.f);
                if (kb < p.Kg) {
                    if (stripe_live) {
                        const uint8_t* blk = p.wq + ((int64_t)nb * p.Kg + kb) * BS + 16 * G;
                        wv.x = h2f(*reinterpret_cast<const uint16_t*>(blk + 2 * lane));
                        if (QTYPE == 1) wv.y = h2f(*reinterpret_cast<const uint16_t*>(blk + 64 + 2 * lane));
                    }
                    const int64_t m = m0 + pt;
                    if (m < p.rows) {
                        xv.x = __ldg(p.xs + m * p.Kg + kb);
                        if (QTYPE == 1) xv.y = __ldg(p.gs + m * p.Kg + kb);
                    }
                }
                wsc[gi * kTileN + pt] = wv;
                xsc[gi * kTileM + pt] = xv;
            }
            fence_proxy_async();  // generic-proxy stores above -> visible to the tensor core's async proxy
            mbar_arrive(bar_full + 8 * s);
        }
    } else if (warp == kMmaWarp) {
        // =================== MMA issue: one elected lane ===================
        if (lane == 0) {
            // instruction descriptor: D = s32, A = u8 (s8 when sign-extended), B = s8, both K-major, N = 128, M = 128
            const uint32_t idesc = (2u << 4) | ((SIGNED ? 1u : 0u) << 7) | (1u << 10) | ((uint32_t)(kTileM >> 3) << 17) |
                                   ((uint32_t)(kTileN >> 4) << 24);
            int gcount = 0;
            bool ok = true;
            for (int it = 0; it < nstage && ok; it++) {
                const int s = it % kStages;
                if (!mbar_wait(bar_full + 8 * s, (it / kStages) & 1, abort_flag)) break;
                tc_fence_after();
                const uint32_t a_base = smem_u32(smem + s * kStageBytes), b_base = a_base + kABytes;
                const int ng = min(GPS, p.Kg - it * GPS);
                for (int gi = 0; gi < ng; gi++, gcount++) {
                    const int b = gcount % kTmemBufs;
                    if (!mbar_wait(bar_tempty + 8 * b, ((gcount / kTmemBufs) & 1) ^ 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t d = tmem_base + b * kTileM;
#pragma unroll
                    for (int ks = 0; ks < MMAS; ks++) {
                        const uint32_t koff = (uint32_t)(gi * G + ks * 32);  // bytes into the 128-byte row
                        tc_mma_i8(d, make_desc(a_base + koff), make_desc(b_base + koff), idesc, ks > 0 ? 1u : 0u);
                    }
                    tc_commit(bar_tfull + 8 * b);  // the group's integers are complete in TMEM
                }
                tc_commit(bar_empty + 8 * s);  // the stage's operands have been consumed
            }
        }
        __syncwarp();
    } else {
        // =================== epilogue: 8 warps ===================
        const int quarter = warp & 3, half = warp >> 2;
        const int nrow = quarter * 32 + lane;  // tile column n handled by this thread (= TMEM lane)
        float acc[64];
#pragma unroll
        for (int i = 0; i < 64; i++) acc[i] = 0.0f;
        int gcount = 0;
        bool ok = true;
        for (int it = 0; it < nstage && ok; it++) {
            const int s = it % kStages;
            const uint8_t* st = smem + s * kStageBytes;
            const float2* wsc = reinterpret_cast<const float2*>(st + kABytes + kBBytes);
            const float4* xsc4 = reinterpret_cast<const float4*>(st + kABytes + kBBytes + kWscBytes);
            const int ng = min(GPS, p.Kg - it * GPS);
            for (int gi = 0; gi < ng; gi++, gcount++) {
                const int b = gcount % kTmemBufs;
                if (!mbar_wait(bar_tfull + 8 * b, (gcount / kTmemBufs) & 1, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const float2 w = wsc[gi * kTileN + nrow];  // wd, wm of this thread's column
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {  // two loads of 32 columns keep the register count down
                    uint32_t v[32];
                    tc_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * kTileM + half * 64 + hh * 32, v);
                    tc_wait_ld();
                    if (hh == 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_tempty + 8 * b);  // the buffer can be overwritten
                    }
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const float4 x2 = xsc4[gi * (kTileM / 2) + half * 32 + hh * 16 + j];  // xs, gs of two rows
                        // exact int -> float: |I| < 2^22, so (I + 0x4B400000) reinterpreted is 12582912 + I
                        const float i0 = __int_as_float((int)v[2 * j] + 0x4B400000) - 12582912.0f;
                        const float i1 = __int_as_float((int)v[2 * j + 1] + 0x4B400000) - 12582912.0f;
                        const int a0 = hh * 32 + 2 * j;
                        acc[a0] = fmaf(__fmul_rn(w.x, x2.x), i0, acc[a0]);
                        acc[a0 + 1] = fmaf(__fmul_rn(w.x, x2.z), i1, acc[a0 + 1]);
                        if (QTYPE == 1) {
                            acc[a0] = fmaf(w.y, x2.y, acc[a0]);
                            acc[a0 + 1] = fmaf(w.y, x2.w, acc[a0 + 1]);
                        }
                    }
                }
            }
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(bar_empty + 8 * s);  // done with the stage's scales
        }
        if (ok) {
            const int64_t n = n0 + nrow;
            if (n < p.N) {
#pragma unroll
                for (int j = 0; j < 64; j++) {
                    const int64_t m = m0 + half * 64 + j;
                    if (m < p.rows) p.y[m * p.ldy + n] = acc[j];
                }
            }
        }
    }

    // ---- teardown: everyone meets, then the allocating warp frees TMEM
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, 0x50524546);  // 'PREF': a bounded wait ran out
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

template <int G, int QTYPE, bool SIGNED>
int launch_prefill_variant(const PrefillParams& p, cudaStream_t s) {
    static bool attr_done[64] = {};
    int dev = 0;
    Q4FC_CUDA_OK(cudaGetDevice(&dev));
    auto* fn = fc_prefill_kernel<G, QTYPE, SIGNED>;
    if (dev < 64 && !attr_done[dev]) {
        Q4FC_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        attr_done[dev] = true;
    }
    const int64_t n_tiles = ((int64_t)p.Ng * 32 + kTileN - 1) / kTileN;
    const int64_t m_tiles = (p.rows + kTileM - 1) / kTileM;
    if (n_tiles > 0x7fffffffLL || m_tiles > 65535) {
        set_error("fc_prefill: %lld x %lld tiles exceed the grid limit", (long long)n_tiles, (long long)m_tiles);
        return Q4FC_ELIMIT;
    }
    fn<<<dim3((unsigned)n_tiles, (unsigned)m_tiles), kThreads, kSmemBytes, s>>>(p);
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

// workspace: [status 256][codes rows x Kp, 256-aligned][xs rows x Kg f32][gs rows x Kg f32]
struct WsLayout {
    size_t codes, xs, gs, total;
};
WsLayout ws_layout(int64_t rows, int64_t Kg, int G) {
    WsLayout l;
    l.codes = kWsStatusBytes;
    l.xs = align_up(l.codes + (size_t)rows * Kg * G, 256);
    l.gs = align_up(l.xs + (size_t)rows * Kg * 4, 256);
    l.total = align_up(l.gs + (size_t)rows * Kg * 4, 256);
    return l;
}

}  // namespace

size_t prefill_workspace_bytes(int64_t rows, int64_t K, int64_t N, int qtype, int G) {
    (void)N, (void)qtype;
    return ws_layout(rows, (K + G - 1) / G, G).total;
}

int launch_fc_prefill(const float* x, int64_t rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng,
                      int64_t Kg, int qtype, int G, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes,
                      unsigned flags, cudaStream_t s) {
    if (rows == 0 || N == 0) return Q4FC_OK;
    const WsLayout l = ws_layout(rows, Kg, G);
    if (ws == nullptr || ws_bytes < l.total) {
        set_error("fc_prefill: workspace of %zu bytes given, %zu needed", ws_bytes, l.total);
        return Q4FC_EWORKSPACE;
    }
    uint8_t* base = static_cast<uint8_t*>(ws);
    PrefillParams p;
    p.wq = wq;
    p.codes = reinterpret_cast<const int8_t*>(base + l.codes);
    p.xs = reinterpret_cast<const float*>(base + l.xs);
    p.gs = reinterpret_cast<const float*>(base + l.gs);
    p.y = y;
    p.status = reinterpret_cast<int*>(base);
    p.rows = rows, p.N = N, p.ldy = ldy, p.Kp = Kg * G;
    p.Ng = (int)Ng, p.Kg = (int)Kg;
    // the reference's 1/16 activation scale of Q4_0 pairs with its x16 nibble shift; neither is materialised
    int rc = launch_quant_x(x, rows, K, ldx, G, 1.0f, reinterpret_cast<int8_t*>(base + l.codes),
                            reinterpret_cast<float*>(base + l.xs), reinterpret_cast<float*>(base + l.gs), s);
    if (rc) return rc;
    const bool sgn = (flags & Q4FC_FLAG_NIBBLE_SIGNED) && qtype == 0;
    if (qtype == 1 && G == 32) return launch_prefill_variant<32, 1, false>(p, s);
    if (qtype == 1 && G == 128) return launch_prefill_variant<128, 1, false>(p, s);
    if (qtype == 0 && G == 32 && !sgn) return launch_prefill_variant<32, 0, false>(p, s);
    if (qtype == 0 && G == 128 && !sgn) return launch_prefill_variant<128, 0, false>(p, s);
    if (qtype == 0 && G == 32) return launch_prefill_variant<32, 0, true>(p, s);
    return launch_prefill_variant<128, 0, true>(p, s);
}

}  // namespace q4fc
