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
// Warp roles (24 warps, 21 of them busy): 0-15 epilogue (warp%4 = TMEM lane quarter, warp/4 =
// which 32 of the 128 tile rows), 16-19 producers (unpack A and stage the
// scales of one 128-k stage: generic-proxy stores + fence.proxy.async; one of
// them also issues the TMA load of the B tile from the code matrix), 20 MMA
// issue (one elected lane).  mbarriers: full/empty per shared-memory stage,
// tfull/tempty per TMEM buffer.  Every wait is bounded: when a wait runs out
// the CTA sets the workspace status word, every role leaves its loop, TMEM is
// freed and the kernel returns.
#include <cuda.h>  // CUtensorMap and the cuTensorMapEncodeTiled prototype (resolved at run time, libcuda is not linked)

#include <atomic>

#include "common.cuh"

namespace q4fc {
namespace {

constexpr int kTileN = 128;            // weight columns per tile = TMEM lanes
constexpr int kTileM = 128;            // activation rows per tile = TMEM columns per buffer
constexpr int kStageK = 128;           // k per shared-memory stage (one 128-byte swizzle row)
constexpr int kStages = 4;
constexpr int kTmemBufs = 4;
constexpr int kEpiWarps = 16, kProdWarps = 4;
constexpr int kProdThreads = kProdWarps * 32;
constexpr int kThreads = (kEpiWarps + kProdWarps + 4) * 32;  // the MMA warp's warpgroup is filled up with idle warps
constexpr int kMmaWarp = kEpiWarps + kProdWarps;
constexpr uint64_t kWaitLimitNs = 1000000000ull;  // every mbarrier wait gives up after one second

// stage layout in shared memory (bytes); A and B tiles are 1024-byte aligned (swizzle atom)
constexpr int kABytes = kTileN * kStageK;          // 16 KB
constexpr int kBBytes = kTileM * kStageK;          // 16 KB
constexpr int kWscBytes = 4 * kTileN * 8;          // [group in stage][n] {wd, wm} fp32
constexpr int kXscBytes = 4 * kTileM * 8;          // [group in stage][row pair] {xs0, xs1, gsum0, gsum1} fp32
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
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// 2-D tiled TMA load (no multicast): box at (x, y) of the tensor map -> shared memory, completion on `bar`
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
// packed fp32 pairs (sm_100): one issue slot for two fused multiply-adds
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
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
__global__ void __launch_bounds__(kThreads, 1) fc_prefill_kernel(const PrefillParams p,
                                                                 const __grid_constant__ CUtensorMap codes_map) {
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
            mbar_init(bar_full + 8 * i, kProdThreads + 1);  // producer threads + the TMA issuer's expect_tx
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

    // Register budget per role (whole warpgroups): the launch gives every thread 80; producers and the
    // MMA warpgroup hand registers back, the epilogue warpgroups take 96 each (what is handed back,
    // 4*32*16 + 4*32*56 = 9216, covers what is taken, 16*32*16 = 8192, so no request can block).
    if (warp >= kEpiWarps && warp < kMmaWarp) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        // =================== producers: one 128-k stage at a time ===================
        const int pt = threadIdx.x - kEpiWarps * 32;  // 0..127
        const int pw = pt >> 5;                       // stripe of the tile handled by this warp
        const int c = lane & 7, rr = lane >> 3;       // 16-byte chunk (columns 4c..4c+3), row inside a 4-row set
        const int nb = nb0 + pw;
        const bool stripe_live = nb < p.Ng;
        // columns are stored in a rotated order so that a half warp covers all 8 swizzle rows
        // (conflict-free 8-byte stores); rows and the rotation do not change from stage to stage
        uint32_t row_off[4];
        int col_of[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            col_of[i] = (i + (c >> 1)) & 3;
            const uint32_t row = pw * 32 + 4 * c + col_of[i];
            row_off[i] = (row >> 3) * 1024 + (row & 7) * 128 + ((row & 7) << 16);  // low half: offset, high half: row&7
        }
        const uint8_t* stripe_base = p.wq + (int64_t)nb * p.Kg * BS;
        const int64_t m_mine = m0 + pt;
        for (int it = 0; it < nstage; it++) {
            const int s = it % kStages;
            if (!mbar_wait(bar_empty + 8 * s, ((it / kStages) & 1) ^ 1, abort_flag)) break;
            uint8_t* st = smem + s * kStageBytes;
            const uint32_t a_base = smem_u32(st), b_base = a_base + kABytes;
            float2* wsc = reinterpret_cast<float2*>(st + kABytes + kBBytes);
            float* xsc = reinterpret_cast<float*>(st + kABytes + kBBytes + kWscBytes);
            const int kb0 = it * GPS;
            if (pt == 0) {  // B: 128 rows x 128 bytes of codes, swizzled by the TMA unit; rows beyond the matrix read 0
                mbar_arrive_expect_tx(bar_full + 8 * s, kBBytes);
                tma_load_2d(b_base, &codes_map, bar_full + 8 * s, it * kStageK, (int)m0);
            }
            // ---- A: unpack nibbles of stripe nb: 16 word-rows (8 k each) x 32 columns
            uint4 w[4];
#pragma unroll
            for (int i4 = 0; i4 < 4; i4++) {
                const int r = 4 * i4 + rr;  // word-row inside the stage: k = 8r .. 8r+7
                w[i4] = make_uint4(0u, 0u, 0u, 0u);
                const int kb = (G == 128) ? kb0 : kb0 + i4;
                if (stripe_live && kb < p.Kg) {
                    const int row_in_block = (G == 128) ? r : rr;
                    w[i4] = ldg_stream_v4(stripe_base + (int64_t)kb * BS + row_in_block * 128 + c * 16);
                }
            }
            // ---- scales of the stage's groups (loads issued before the unpack stores)
            float2 wv[GPS];
            float xv[GPS], gv[GPS];
#pragma unroll
            for (int gi = 0; gi < GPS; gi++) {
                const int kb = kb0 + gi;
                wv[gi] = make_float2(0.f, 0.f);
                xv[gi] = 0.f, gv[gi] = 0.f;
                if (kb < p.Kg) {
                    if (stripe_live) {
                        const uint8_t* tail = stripe_base + (int64_t)kb * BS + 16 * G;
                        wv[gi].x = h2f(*reinterpret_cast<const uint16_t*>(tail + 2 * lane));
                        if (QTYPE == 1) wv[gi].y = h2f(*reinterpret_cast<const uint16_t*>(tail + 64 + 2 * lane));
                    }
                    if (m_mine < p.rows) {
                        xv[gi] = __ldg(p.xs + m_mine * p.Kg + kb);
                        if (QTYPE == 1) gv[gi] = __ldg(p.gs + m_mine * p.Kg + kb);
                    }
                }
            }
#pragma unroll
            for (int i4 = 0; i4 < 4; i4++) {
                const int r = 4 * i4 + rr;
                const uint32_t chunk = (uint32_t)(r >> 1), sub = (uint32_t)(r & 1) * 8;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t word = col_of[i] == 0 ? w[i4].x : col_of[i] == 1 ? w[i4].y : col_of[i] == 2 ? w[i4].z : w[i4].w;
                    uint32_t lo = word & 0x0F0F0F0Fu, hi = (word >> 4) & 0x0F0F0F0Fu;
                    if (SIGNED) {  // sign-extend each nibble into its byte
                        lo |= (lo & 0x08080808u) * 0x1Eu;
                        hi |= (hi & 0x08080808u) * 0x1Eu;
                    }
                    const uint32_t addr = a_base + (row_off[i] & 0xFFFFu) + (((chunk ^ (row_off[i] >> 16)) & 7) << 4) + sub;
                    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(lo), "r"(hi) : "memory");
                }
            }
#pragma unroll
            for (int gi = 0; gi < GPS; gi++) {
                wsc[gi * kTileN + pt] = wv[gi];
                // row pairs are kept as {xs0, xs1, gs0, gs1} for the packed epilogue arithmetic
                float* q = xsc + (gi * (kTileM / 2) + (pt >> 1)) * 4 + (pt & 1);
                q[0] = xv[gi];
                q[2] = gv[gi];
            }
            fence_proxy_async();  // generic-proxy stores above -> visible to the tensor core's async proxy
            mbar_arrive(bar_full + 8 * s);
        }
    } else if (warp >= kMmaWarp) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
        // =================== MMA issue: one elected lane of one warp ===================
        if (warp == kMmaWarp && lane == 0) {
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
        asm volatile("setmaxnreg.inc.sync.aligned.u32 96;");
        // =================== epilogue: 16 warps, 32 lanes x 32 columns each ===================
        const int quarter = warp & 3, cgrp = warp >> 2;
        const int nrow = quarter * 32 + lane;  // tile column n handled by this thread (= TMEM lane)
        uint64_t acc[16];                      // 32 fp32 accumulators as 16 packed pairs (rows 2j, 2j+1)
#pragma unroll
        for (int i = 0; i < 16; i++) acc[i] = 0ull;
        const uint64_t neg_magic = pack2(-12582912.0f, -12582912.0f);
        int gcount = 0;
        bool ok = true;
        for (int it = 0; it < nstage && ok; it++) {
            const int s = it % kStages;
            const uint8_t* st = smem + s * kStageBytes;
            const float2* wsc = reinterpret_cast<const float2*>(st + kABytes + kBBytes);
            const ulonglong2* xsc2 = reinterpret_cast<const ulonglong2*>(st + kABytes + kBBytes + kWscBytes);
            const int ng = min(GPS, p.Kg - it * GPS);
            for (int gi = 0; gi < ng; gi++, gcount++) {
                const int b = gcount % kTmemBufs;
                if (!mbar_wait(bar_tfull + 8 * b, (gcount / kTmemBufs) & 1, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                uint32_t v[32];
                tc_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * kTileM + cgrp * 32, v);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * b);  // the buffer can be overwritten
                const float2 w = wsc[gi * kTileN + nrow];          // wd, wm of this thread's column
                const uint64_t wd2 = pack2(w.x, w.x), wm2 = pack2(w.y, w.y);
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const ulonglong2 xg = xsc2[gi * (kTileM / 2) + cgrp * 16 + j];  // {xs0, xs1}, {gs0, gs1}
                    // exact int -> float: |I| < 2^22, so (I + 0x4B400000) reinterpreted is 12582912 + I
                    const uint64_t i2 = fadd2(pack2(__int_as_float((int)v[2 * j] + 0x4B400000),
                                                    __int_as_float((int)v[2 * j + 1] + 0x4B400000)),
                                              neg_magic);
                    acc[j] = ffma2(fmul2(wd2, xg.x), i2, acc[j]);
                    if (QTYPE == 1) acc[j] = ffma2(wm2, xg.y, acc[j]);
                }
            }
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(bar_empty + 8 * s);  // done with the stage's scales
        }
        if (ok) {
            const int64_t n = n0 + nrow;
            if (n < p.N) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int64_t m = m0 + cgrp * 32 + 2 * j;
                    float lo, hi;
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[j]));
                    if (m < p.rows) p.y[m * p.ldy + n] = lo;
                    if (m + 1 < p.rows) p.y[(m + 1) * p.ldy + n] = hi;
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

// cuTensorMapEncodeTiled, looked up once through the runtime (the driver library is not linked)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    // a function-local static is initialised once, also when several host threads arrive together
    static const EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(sym);
        cudaGetLastError();
        return static_cast<EncodeTiledFn>(nullptr);
    }();
    return fn;
}

// the code matrix [rows][Kp] int8 as a 2-D tensor; boxes of 128 bytes x 128 rows land in the
// 128-byte-swizzle layout that the MMA descriptors describe; out-of-range rows and k read as 0
int make_codes_map(CUtensorMap* map, const int8_t* codes, int64_t rows, int64_t Kp) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) {
        set_error("fc_prefill: cuTensorMapEncodeTiled is not available from this driver");
        return Q4FC_ECUDA;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)Kp, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)Kp};
    const cuuint32_t box[2] = {(cuuint32_t)kStageK, (cuuint32_t)kTileM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(codes), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("fc_prefill: cuTensorMapEncodeTiled failed with %d (rows=%lld, Kp=%lld)", (int)r, (long long)rows,
                  (long long)Kp);
        return Q4FC_ECUDA;
    }
    return Q4FC_OK;
}

template <int G, int QTYPE, bool SIGNED>
int launch_prefill_variant(const PrefillParams& p, const CUtensorMap& map, cudaStream_t s) {
    static std::atomic<bool> attr_done[64] = {};  // set once per device; a second setter repeats the same call
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
    fn<<<dim3((unsigned)n_tiles, (unsigned)m_tiles), kThreads, kSmemBytes, s>>>(p, map);
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

// workspace: [status 256][what the decode kernels keep between calls: decode_prequant_offset() bytes]
//            [codes rows x Kp, 256-aligned][xs rows x Kg f32][gs rows x Kg f32]
// The quantized activations start where the decode path's own quantizer scratch starts: calls on one
// workspace are ordered, so the two can share that space, and neither lands on the stream-K stripe
// counters, which must stay zero between calls.
struct WsLayout {
    size_t codes, xs, gs, total;
};
WsLayout ws_layout(int64_t rows, int64_t Kg, int G) {
    WsLayout l;
    l.codes = decode_prequant_offset();
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
    if (rows > 0x7fffffffLL || p.Kp > 0x7fffffffLL) {
        set_error("fc_prefill: rows=%lld or K=%lld beyond the 2^31 coordinate range", (long long)rows, (long long)K);
        return Q4FC_ELIMIT;
    }
    CUtensorMap map;
    rc = make_codes_map(&map, p.codes, rows, p.Kp);
    if (rc) return rc;
    const bool sgn = (flags & Q4FC_FLAG_NIBBLE_SIGNED) && qtype == 0;
    if (qtype == 1 && G == 32) return launch_prefill_variant<32, 1, false>(p, map, s);
    if (qtype == 1 && G == 128) return launch_prefill_variant<128, 1, false>(p, map, s);
    if (qtype == 0 && G == 32 && !sgn) return launch_prefill_variant<32, 0, false>(p, map, s);
    if (qtype == 0 && G == 128 && !sgn) return launch_prefill_variant<128, 0, false>(p, map, s);
    if (qtype == 0 && G == 32) return launch_prefill_variant<32, 0, true>(p, map, s);
    return launch_prefill_variant<128, 0, true>(p, map, s);
}

}  // namespace q4fc
