// A chain of dependent decode FCs in ONE launch: the per-token FC schedule of the reference's Model.forward
// (chatllama/main.py:331-380 -- per layer q, k, v | o | gate, up | down, then lm_head; 225 fc_Q4A calls for 32
// layers, each fed by the one before through rmsnorm / iadd / silu * up) as a persistent kernel.
//
// Why one launch.  A decode FC reads megabytes of weights and a few kilobytes of activations.  As separate launches
// every FC pays a start (barriers, first copies: a couple of microseconds during which HBM idles) and an end (the
// slowest CTA), and the next one cannot start before its input exists.  Only the ACTIVATIONS depend on the step
// before; the weights never do.  Here one CTA per SM lives for the whole token: its producer thread walks the
// CTA's share of every step's stripes and keeps a shared-memory ring of weight blocks full with 1-D bulk copies
// (cp.async.bulk, global -> shared, completion on an mbarrier), never waiting for anything but a free slot, while
// the 16 consumer warps go step by step: grid barrier (the outputs of the step before are complete), quantize the
// step's input into shared memory -- with the transform the reference applies between the FCs -- then
// mma.sync.m16n8k32 (u8 x s8) over the blocks in the ring, partial sums through shared memory, outputs to global.
// While the consumers sit in a barrier or quantize, the ring (up to ~200 KB) keeps filling, so the weight stream
// does not wait for a dependency.  What bounds a step is then the consumers' own sequence -- barrier, input from L2,
// quantization, arithmetic, partial sums, outputs -- which nothing overlaps: with one activation row and a few tens
// of megabytes per step that sequence, not HBM, sets the pace.
//
// Steps.  A step is one input (fp32 [rows][ldx], rows <= 8, written by an earlier step or by the caller before the
// launch), a transform, and one or more jobs (weight tensors) on it:
//   PLAIN      the input as it is                                (FC_dynamic_quantize_x, ops/op_fc.hpp:221-272)
//   RMSNORM    (x * 1/sqrt(mean(x^2) + eps)) * w                 (llmops.rmsnorm, ops/op_misc.hpp:142-181)
//   SILU_MUL   up * silu(x)                                      (llmops.itrans + imul, ops/op_misc.hpp:83-138)
// and per job an optional addend on the output (llmops.iadd: bias or residual stream).  Codes, scales, sums and
// FC arithmetic are the shared pieces of decode_math.cuh, so a PLAIN or SILU_MUL step has the codes of the stand-alone
// launches (q4fc_quant_x_q8 / q4fc_silu_mul_quant) bit for bit and the outputs of q4fc_fc_decode_multi within the
// rounding of the fp32 sums.  RMSNORM adds the squares in tree order, not in the reference's eight sequential chains
// (ops/utils.hpp:92-98; a microsecond of dependent fma that every SM would repeat at every step): the factor
// 1/sqrt(..) can differ from q4fc_rmsnorm_quant's in its last place, the normalized values by one ulp.
//
// Work split.  Step s has S_s stripes (32 output columns, Kg contiguous blocks); CTA c takes the contiguous range
// [c' S_s / P, (c'+1) S_s / P) with c' = (c + rot_s) mod P: rot_s moves round so that the CTAs that get one stripe
// more (or none) differ from step to step.
//
// Step barrier.  Cooperative launch (all CTAs resident).  Every step has an arrival counter of its own in global
// memory (one 128-byte line each), never reset: the warp that stores a (stripe, row) of step s adds one with release
// semantics right behind its stores; a CTA that needs the outputs of step s polls the counter until it reaches
// (launches so far + 1) x (stripes x rows of step s).  "Launches so far" is a word the last CTA to leave
// increments, so a handle can be launched again and again (and replayed from a CUDA graph) with nothing to reset.
// Every wait -- this one and the mbarrier waits -- is bounded by one second of %globaltimer: when it runs out the
// status word is set, the CTA's other waits end at once, all loops run to their ends and the kernel returns.  The
// host clears the counters when it reads a non-zero status.
#include <mutex>
#include <vector>

#include "common.cuh"
#include "decode_math.cuh"
#include "ring_ptx.cuh"

namespace q4fc {
namespace {

constexpr int kCW = 16;  // consumer warps
constexpr int kCThreads = (kCW + 1) * 32;
constexpr int kCRingMax = 10;
constexpr int kCPartBufs = 4;
constexpr int kChainAhead = 4;  // slots of the next step the producer requests before the consumers get there

// The tables of a chain (a few KB) are copied into every CTA's shared memory at the start: a table read on the
// critical path of a step then costs a shared-memory access, not an L2 round trip.
struct ChainJobDev {
    const uint8_t* wq;
    float* y;
    const float* addend;
    int N, ldy, addend_ld;
    int s_end;  // one past this job's last stripe, counted inside its step
};
struct ChainStepDev {
    const float* x;
    const float* aux;  // RMSNORM: weight [K]; SILU_MUL: the `up` rows, same layout as x
    int ldx, K;
    float eps;
    int transform;
    int Kg;
    int job0, stripes;
    int rot;
    int units;  // arrivals a launch adds to the step's counter: its stripes x rows
    int pad;
};
static_assert(sizeof(ChainJobDev) % 8 == 0 && sizeof(ChainStepDev) % 8 == 0, "tables are copied as 8-byte words");
constexpr size_t kChainTableMax = 40 * 1024;  // most table bytes a chain may have (they share the SM with the ring)

struct ChainParams {
    const ChainStepDev* steps;  // then the jobs: one allocation, table_bytes in all
    const ChainJobDev* jobs;
    int nsteps, table_bytes, part_off;
    int rows, rows_p;
    int code_stride, kg_max;
    int depth, slot_bytes, ring_off;
    unsigned* arrivals;  // [nsteps] counters, 32 words (128 bytes) apart, monotonic over launches
    unsigned* launches;  // completed launches of this handle
    unsigned* leavers;   // CTAs of the current launch that are done
    int* status;
};

template <int G, int QTYPE>
struct ChainShape {
    static constexpr int BS = block_bytes(QTYPE, G);
    static constexpr int SETS = G / 32;
    static constexpr int NBLK = (G == 32) ? 4 : 1;
    static constexpr int SB = kCW * NBLK;
};

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* a) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a) : "memory");
    return v;
}

// arrive (one lane of the warp that stored the outputs, behind a __syncwarp): a release at GPU scope -- the warp's
// stores are visible to whoever then reads the count with an acquire.  wait (one thread per CTA): until `target`
// arrivals are in (wrap-safe comparison).  No fence.sc anywhere: the weights an SM has cached stay cached.
__device__ __forceinline__ void step_arrive(unsigned* counter) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
}
__device__ __forceinline__ void step_wait(const unsigned* counter, unsigned target, const ChainParams& p, volatile int* fail) {
    if ((int)(ld_acquire_gpu(counter) - target) >= 0 || *fail != 0) return;
    const unsigned long long t0 = globaltimer_ns();
    for (unsigned it = 1; (int)(ld_acquire_gpu(counter) - target) < 0; it++) {
        if ((it & 63) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
            *fail = 1;
            atomicCAS(p.status, 0, 0x43474252);  // 'CGBR'
            return;
        }
    }
}

// The consumer warps quantize the step's input rows (all K) into shared memory.  Item = one 128-k chunk of up to RI
// rows.  A warp works on CH items at a time as independent rows of one straight-line call (their shuffle and divide
// chains overlap) and requests the next CH items before it starts on the present ones, so a step costs one L2 round
// trip, not one per item.  The code is kept compact on purpose (one loop, no unrolling over items): it runs once per
// step, cold, and a step's time is partly the time to fetch its instructions.  `scratch`: 64 floats nobody else
// uses meanwhile.
template <int G, int ROWS>
__device__ __noinline__ void chain_quantize(const ChainStepDev* __restrict__ Sp, int rows, int warp, int lane,
                                            uint8_t* codes, float* sc, int code_stride, float* scratch) {
    constexpr int SEG = G / 4;
    constexpr int GPC = 128 / G;
    constexpr int RI = ROWS > 4 ? 4 : ROWS;
    constexpr int RGRP = ROWS / RI;  // 1 or 2: warp w always works on row group w % RGRP (kCW is even)
    constexpr int CH = RI == 1 ? 2 : 1;
    const float* x = Sp->x;  // (shared memory: the CTA's copy of the table)
    const float* aux_p = Sp->aux;
    const int64_t K = Sp->K, ldx = Sp->ldx;
    const int Kg = Sp->Kg, transform = Sp->transform;
    const float eps = Sp->eps;
    const int chunks = (int)(((int64_t)Kg * G + 127) >> 7);
    const int items = chunks * RGRP;
    const int m0 = (warp % RGRP) * RI;
    const bool single = items <= kCW * CH;  // every warp holds all of its items at once

    auto load = [&](float (&v)[CH][RI][4], float (&u)[CH][RI][4], int item0, bool with_aux) {
#pragma unroll
        for (int ib = 0; ib < CH; ib++) {
            const int item = item0 + ib * kCW;
            const int64_t e = (int64_t)(item / RGRP) * 128 + lane * 4;
#pragma unroll
            for (int mm = 0; mm < RI; mm++) {
                const int m = m0 + mm;
                v[ib][mm][0] = v[ib][mm][1] = v[ib][mm][2] = v[ib][mm][3] = 0.0f;
                u[ib][mm][0] = u[ib][mm][1] = u[ib][mm][2] = u[ib][mm][3] = 0.0f;
                if (item < items && m < rows && e + 4 <= K) {  // K % 8 == 0: a lane's four values exist together
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(x + m * ldx + e));
                    v[ib][mm][0] = a.x, v[ib][mm][1] = a.y, v[ib][mm][2] = a.z, v[ib][mm][3] = a.w;
                    if (with_aux && transform == Q4FC_CHAIN_SILU_MUL) {
                        const float4 b = __ldcg(reinterpret_cast<const float4*>(aux_p + m * ldx + e));
                        u[ib][mm][0] = b.x, u[ib][mm][1] = b.y, u[ib][mm][2] = b.z, u[ib][mm][3] = b.w;
                    } else if (with_aux && transform == Q4FC_CHAIN_RMSNORM) {
                        const float4 b = __ldg(reinterpret_cast<const float4*>(aux_p + e));
                        u[ib][mm][0] = b.x, u[ib][mm][1] = b.y, u[ib][mm][2] = b.z, u[ib][mm][3] = b.w;
                    }
                }
            }
        }
    };

    float v[CH][RI][4], u[CH][RI][4];
    float r[RI];
#pragma unroll
    for (int mm = 0; mm < RI; mm++) r[mm] = 0.0f;
    if (transform == Q4FC_CHAIN_RMSNORM) {
        // 1 / sqrt(mean(x^2) + eps).  The sum of squares is tree-ordered (lane sums, butterfly, warps in order): fixed
        // order, the same from run to run, but not the reference's eight sequential chains (ops/utils.hpp:92-98),
        // which cost a microsecond of dependent fma per step on every SM -- the factor can differ from the
        // reference's in its last place.
        float ss[RI];
#pragma unroll
        for (int mm = 0; mm < RI; mm++) ss[mm] = 0.0f;
#pragma unroll 1
        for (int item0 = warp; item0 < items; item0 += kCW * CH) {
            load(v, u, item0, single);
#pragma unroll
            for (int ib = 0; ib < CH; ib++)
#pragma unroll
                for (int mm = 0; mm < RI; mm++)
#pragma unroll
                    for (int jj = 0; jj < 4; jj++) ss[mm] = __fmaf_rn(v[ib][mm][jj], v[ib][mm][jj], ss[mm]);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
#pragma unroll
            for (int mm = 0; mm < RI; mm++) ss[mm] += __shfl_xor_sync(0xffffffffu, ss[mm], off);
        if (lane == 0) {
#pragma unroll
            for (int mm = 0; mm < RI; mm++) scratch[warp * 4 + mm] = ss[mm];
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory");
#pragma unroll
        for (int mm = 0; mm < RI; mm++) {
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < kCW / RGRP; w++) tot = __fadd_rn(tot, scratch[(w * RGRP + warp % RGRP) * 4 + mm]);
            const float rms = __fdiv_rn(tot, (float)K);
            r[mm] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(rms, eps)));
        }
    }
    if (!(transform == Q4FC_CHAIN_RMSNORM && single)) load(v, u, warp, true);
#pragma unroll 1
    for (int item0 = warp; item0 < items; item0 += kCW * CH) {
        float vn[CH][RI][4], un[CH][RI][4];
        const bool more = item0 + kCW * CH < items;
        if (more) load(vn, un, item0 + kCW * CH, true);  // on its way while the present items are worked on
        int lens[CH * RI];
#pragma unroll
        for (int ib = 0; ib < CH; ib++) {
            const int item = item0 + ib * kCW;
            const int kbl = (item / RGRP) * GPC + lane / SEG;
            const int len = (item < items && kbl < Kg) ? (int)min((int64_t)G, K - (int64_t)kbl * G) : 0;
#pragma unroll
            for (int mm = 0; mm < RI; mm++) {
                lens[ib * RI + mm] = len;
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    const float val = v[ib][mm][jj];
                    if (transform == Q4FC_CHAIN_SILU_MUL) {
                        const float sg = __fdiv_rn(val, __fadd_rn(1.0f, expf(-val)));
                        v[ib][mm][jj] = __fmul_rn(u[ib][mm][jj], sg);
                    } else if (transform == Q4FC_CHAIN_RMSNORM) {
                        v[ib][mm][jj] = __fmul_rn(__fmul_rn(val, r[mm]), u[ib][mm][jj]);
                    }
                }
            }
        }
        uint32_t packed[CH * RI];
        float d[CH * RI], aux[CH * RI];
        q8_quantize_rows_v<G, CH * RI, false>(reinterpret_cast<const float(&)[CH * RI][4]>(v), lane, lens, packed, d, aux);
#pragma unroll
        for (int ib = 0; ib < CH; ib++) {
            const int item = item0 + ib * kCW;
            const int ch = item / RGRP;
            const int kbl = ch * GPC + lane / SEG;
            if (item < items && kbl < Kg) {
                const int64_t e = (int64_t)ch * 128 + lane * 4;
#pragma unroll
                for (int mm = 0; mm < RI; mm++) {
                    const int m = m0 + mm;
                    if (m < rows) {
                        *reinterpret_cast<uint32_t*>(codes + m * code_stride + e) = packed[ib * RI + mm];
                        if (lane % SEG == 0)
                            *reinterpret_cast<float2*>(sc + kbl * 16 + m * 2) = make_float2(d[ib * RI + mm], aux[ib * RI + mm]);
                    }
                }
            }
        }
        if (more) {
#pragma unroll
            for (int ib = 0; ib < CH; ib++)
#pragma unroll
                for (int mm = 0; mm < RI; mm++)
#pragma unroll
                    for (int jj = 0; jj < 4; jj++) v[ib][mm][jj] = vn[ib][mm][jj], u[ib][mm][jj] = un[ib][mm][jj];
        }
    }
}

template <int G, int QTYPE, int ROWS>
__global__ void __launch_bounds__(kCThreads, 1) fc_chain_kernel(const __grid_constant__ ChainParams p) {
    using S_ = ChainShape<G, QTYPE>;
    constexpr int BS = S_::BS;
    constexpr int SETS = S_::SETS;
    constexpr int NBLK = S_::NBLK;
    constexpr int SB = S_::SB;

    extern __shared__ __align__(128) uint8_t smem[];
    // [0,512): mbarriers full[kCRingMax] at 0, empty[kCRingMax] at 80; failure flag at 192;
    // pfull[kCPartBufs] at 256, pfree[kCPartBufs] at 320; then the step and job tables | part [kCPartBufs][kCW][rows_p*32] f32 |
    // sc [kg_max][16] f32 | codes [rows][code_stride] | ring [depth][slot_bytes]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int P = (int)gridDim.x, c = (int)blockIdx.x;
    const int rows = p.rows;
    const int slot_f = p.rows_p * 32;
    const int depth = p.depth;

    const uint32_t bar0 = smem_u32(smem);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kCRingMax + s); };
    auto pfull_bar = [&](int b) { return bar0 + 256u + 8u * b; };
    auto pfree_bar = [&](int b) { return bar0 + 320u + 8u * b; };
    volatile int* fail = reinterpret_cast<volatile int*>(smem + 192);
    volatile int* ready_step = reinterpret_cast<volatile int*>(smem + 200);  // steps whose input this CTA has quantized
    const ChainStepDev* steps = reinterpret_cast<const ChainStepDev*>(smem + 512);
    const ChainJobDev* jobs = reinterpret_cast<const ChainJobDev*>(smem + 512 + sizeof(ChainStepDev) * p.nsteps);
    float* part = reinterpret_cast<float*>(smem + p.part_off);
    float* sc = part + kCPartBufs * kCW * slot_f;
    uint8_t* codes = reinterpret_cast<uint8_t*>(sc + p.kg_max * 16);
    uint8_t* ring = smem + p.ring_off;

    if (threadIdx.x == kCW * 32) {
        for (int i = 0; i < depth; i++) {
            mbar_init(full_bar(i), 1);
            mbar_init(empty_bar(i), kCW);
        }
        for (int i = 0; i < kCPartBufs; i++) {
            mbar_init(pfull_bar(i), kCW);
            mbar_init(pfree_bar(i), rows);
        }
        *fail = 0;
        *ready_step = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    {
        const unsigned long long* src = reinterpret_cast<const unsigned long long*>(p.steps);
        unsigned long long* dst = reinterpret_cast<unsigned long long*>(smem + 512);
        for (int i = threadIdx.x; i < p.table_bytes / 8; i += kCThreads) dst[i] = __ldg(src + i);
    }
    __syncthreads();

    // this CTA's stripes of a step
    auto range = [&](int rot, int stripes, int& a, int& b) {
        int cc = c + rot;
        if (cc >= P) cc -= P;
        a = (int)(((int64_t)cc * stripes) / P);
        b = (int)(((int64_t)(cc + 1) * stripes) / P);
    };

    if (warp == kCW) {
        // ---- producer: the CTA's weight stream over all steps, as far ahead as the ring allows
        if (lane == 0) {
            int s = 0;          // next slot
            uint32_t eph = 1;   // parity of the slot's release to wait for (nothing to wait for in the first round)
            bool first = true;  // the first round through the ring finds every slot free
            for (int st = 0; st < p.nsteps; st++) {
                const ChainStepDev* Sp = steps + st;
                const int Kg = Sp->Kg, job0 = Sp->job0;
                int a, b;
                range(Sp->rot, Sp->stripes, a, b);
                int jb = job0;
                int ahead = 0;  // slots of this step issued before its input is quantized
                for (int sg = a; sg < b; sg++) {
                    while (sg >= jobs[jb].s_end) jb++;
                    const int ls = sg - (jb > job0 ? jobs[jb - 1].s_end : 0);
                    const uint8_t* base = jobs[jb].wq + (int64_t)ls * Kg * BS;
                    for (int kb = 0; kb < Kg; kb += SB) {
                        // No more than kChainAhead slots of a step are requested while the consumers are still on
                        // their way to it: a ring-full of copies from every SM at once keeps HBM and the L2 queues
                        // busy for microseconds, and the few loads and the counter traffic of the step change -- the
                        // sequence that bounds a step -- would wait behind them.
                        if (st > 0 && ahead >= kChainAhead && *ready_step < st) {
                            const unsigned long long t0 = globaltimer_ns();
                            for (unsigned it = 1; *ready_step < st && *fail == 0; it++) {
                                __nanosleep(64);
                                if ((it & 255) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
                                    *fail = 1;
                                    atomicCAS(p.status, 0, 0x43524459);  // 'CRDY'
                                }
                            }
                        }
                        ahead++;
                        // a slot is reused once all consumer warps have taken their blocks out of it
                        if (!first) mbar_wait(empty_bar(s), eph, fail, p.status, 0x43454D50);  // 'CEMP'
                        const uint32_t bytes = (uint32_t)min(SB, Kg - kb) * BS;
                        mbar_expect_tx(full_bar(s), bytes);
                        bulk_g2s(smem_u32(ring + (size_t)s * p.slot_bytes), base + (int64_t)kb * BS, bytes, full_bar(s));
                        if (++s == depth) s = 0, eph ^= 1, first = false;
                    }
                }
            }
        }
    } else {
        unsigned epoch = 0;  // launches of this handle completed before this one
        if (threadIdx.x == 0) epoch = ld_acquire_gpu(p.launches);
        int prev_units = 0;
        const uint8_t* my_codes = codes + g * p.code_stride + 8 * t;
        const bool row_live = g < rows;
        int cs_ = 0;       // ring position
        uint32_t fph = 0;  // parity of the slot's filling to wait for
        int lc = 0;        // stripes finished so far: turns the partial-sum buffers and the adding duty
        for (int st = 0; st < p.nsteps; st++) {
            const ChainStepDev* Sp = steps + st;
            const int Kg = Sp->Kg, job0 = Sp->job0, units = Sp->units;
            int a, b;
            range(Sp->rot, Sp->stripes, a, b);
            const int need = prev_units;
            prev_units = units;
            if (b <= a) continue;
            if (st > 0) {
                // before this CTA reads the step's input, every (stripe, row) of the step before has been stored and
                // counted by the warp that stored it; the CTA barrier also says that all warps here are done with the
                // codes of the step before
                if (threadIdx.x == 0) step_wait(p.arrivals + 32 * (st - 1), (epoch + 1u) * (unsigned)need, p, fail);
                asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory");
            }
            chain_quantize<G, ROWS>(Sp, rows, warp, lane, codes, sc, p.code_stride, part);
            asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory");
            if (threadIdx.x == 0) *ready_step = st;  // the producer may now request the whole ring

            int jb = job0;
            for (int sg = a; sg < b; sg++, lc++) {
                while (sg >= jobs[jb].s_end) jb++;
                const int ls = sg - (jb > job0 ? jobs[jb - 1].s_end : 0);
                float acc[4][2];
#pragma unroll
                for (int i = 0; i < 4; i++) acc[i][0] = acc[i][1] = 0.0f;
                // the row this warp adds at the end of the stripe, if any; its addend (a residual stream written earlier
                // in this launch by other SMs: read from L2) is on its way while the blocks are worked on
                const int m = ((warp - lc * rows) % kCW + kCW) % kCW;
                const ChainJobDev& J = jobs[jb];
                const int64_t n = (int64_t)ls * 32 + lane;
                float addend = 0.0f;
                if (m < rows && n < J.N && J.addend != nullptr) addend = __ldcg(J.addend + m * J.addend_ld + n);
                for (int kb0 = 0; kb0 < Kg; kb0 += SB) {
                    mbar_wait(full_bar(cs_), fph, fail, p.status, 0x4346554C);  // 'CFUL'
                    const int nblk = min(SB, Kg - kb0);
                    const uint8_t* slot = ring + (size_t)cs_ * p.slot_bytes;
                    // this warp's block(s) into registers, the slot handed back, then the arithmetic
                    uint4 q[NBLK][SETS];
                    uint2 wd[NBLK], wm[NBLK];
#pragma unroll
                    for (int i = 0; i < NBLK; i++) {
                        const int bi = warp * NBLK + i;
                        wd[i] = wm[i] = make_uint2(0u, 0u);
                        if (bi < nblk) {
                            const uint8_t* blk = slot + bi * BS;
                            // block rows are 128 bytes apart: two 64-bit loads whose halves swap with the parity of t
                            // cost half the bank conflicts of one 128-bit load
#pragma unroll
                            for (int jj = 0; jj < SETS; jj++) {
                                const uint8_t* rowp = blk + (4 * jj + t) * 128 + g * 16;
                                const bool odd = t & 1;
                                const uint2 u = *reinterpret_cast<const uint2*>(rowp + (odd ? 8 : 0));
                                const uint2 v = *reinterpret_cast<const uint2*>(rowp + (odd ? 0 : 8));
                                q[i][jj] = make_uint4(odd ? v.x : u.x, odd ? v.y : u.y, odd ? u.x : v.x, odd ? u.y : v.y);
                            }
                            wd[i] = *reinterpret_cast<const uint2*>(blk + 16 * G + g * 8);
                            if (QTYPE == 1) wm[i] = *reinterpret_cast<const uint2*>(blk + 16 * G + 64 + g * 8);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_bar(cs_));
#pragma unroll
                    for (int i = 0; i < NBLK; i++) {
                        const int bi = warp * NBLK + i;
                        if (bi < nblk) {
                            const int ck = kb0 + bi;
                            block_accumulate<G, QTYPE, false, (ROWS == 1 ? 1 : 2)>(q[i], wd[i], wm[i], my_codes + ck * G,
                                                                                   row_live, sc + ck * 16, t, acc);
                        }
                    }
                    if (++cs_ == depth) cs_ = 0, fph ^= 1;
                }
                // the warps' partial sums of the stripe meet in shared memory (kCPartBufs buffers in turn); row m is
                // added, in warp order, by warp (lc * rows + m) mod kCW
                const int buf = lc % kCPartBufs;
                const uint32_t use = (uint32_t)(lc / kCPartBufs);
                if (use > 0) mbar_wait(pfree_bar(buf), (use - 1) & 1, fail, p.status, 0x43504652);  // 'CPFR'
                float* pw = part + (buf * kCW + warp) * slot_f;
#pragma unroll
                for (int mi = 0; mi < 2; mi++)
                    if ((2 * t + mi) < p.rows_p)
                        *reinterpret_cast<float4*>(pw + (2 * t + mi) * 32 + g * 4) =
                            make_float4(acc[0][mi], acc[1][mi], acc[2][mi], acc[3][mi]);
                __syncwarp();
                if (lane == 0) mbar_arrive(pfull_bar(buf));
                if (m < rows) {
                    mbar_wait(pfull_bar(buf), use & 1, fail, p.status, 0x43504655);  // 'CPFU'
                    const float* src = part + buf * kCW * slot_f + m * 32 + lane;
                    float sum = src[0];
#pragma unroll
                    for (int w = 1; w < kCW; w++) sum += src[w * slot_f];
                    __syncwarp();
                    if (lane == 0) mbar_arrive(pfree_bar(buf));
                    if (n < J.N) {
                        if (J.addend != nullptr) sum = __fadd_rn(sum, addend);
                        J.y[m * J.ldy + n] = sum;
                    }
                    // this (stripe, row) is out: counted with a release by the warp that stored it, so the count
                    // costs nobody else a barrier and overlaps the other warps' work
                    __syncwarp();
                    if (lane == 0 && st + 1 < p.nsteps) step_arrive(p.arrivals + 32 * st);
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // the last CTA to leave counts the launch: by then every CTA has read the old count
        if (atomicAdd(p.leavers, 1u) == (unsigned)P - 1) {
            atomicExch(p.leavers, 0u);
            __threadfence();
            atomicAdd(p.launches, 1u);
        }
    }
    if (*fail != 0) {
        // a wait ran out: give bulk copies that may still be in flight time to land before the shared memory is
        // handed to another CTA
        for (int i = 0; i < 64; i++) __nanosleep(32000);
    }
}

struct ChainHandle {
    ChainParams p;
    void* dev;  // one allocation: steps, jobs, barrier words, status
    const void* fn;
    int device, grid;
    size_t smem, sync_bytes;
};

std::mutex g_chain_mutex;

template <int G, int QTYPE>
const void* chain_fn_for_rows(int rows) {
    if (rows <= 1) return reinterpret_cast<const void*>(&fc_chain_kernel<G, QTYPE, 1>);
    if (rows <= 2) return reinterpret_cast<const void*>(&fc_chain_kernel<G, QTYPE, 2>);
    if (rows <= 4) return reinterpret_cast<const void*>(&fc_chain_kernel<G, QTYPE, 4>);
    return reinterpret_cast<const void*>(&fc_chain_kernel<G, QTYPE, 8>);
}

}  // namespace

int chain_create(const q4fc_chain_step* steps, int nsteps, const q4fc_fc_job* jobs, int njobs, int rows, int qtype, int G,
                 void** out) {
    const DeviceInfo* di = device_info();
    if (!di) return Q4FC_ECUDA;
    const int BS = block_bytes(qtype, G);
    const int SB = kCW * (G == 32 ? 4 : 1);
    std::vector<ChainStepDev> hs((size_t)nsteps);
    std::vector<ChainJobDev> hj((size_t)njobs);
    int jcur = 0, kg_max = 0;
    // the CTAs that get one stripe more (or none) move round by a stride that shares no factor with the CTA count
    int rot_step = di->sm_count * 3 / 8 | 1;
    auto gcd = [](int a, int b) {
        while (b) {
            const int t = a % b;
            a = b, b = t;
        }
        return a;
    };
    while (gcd(rot_step, di->sm_count) != 1) rot_step += 2;
    for (int s = 0; s < nsteps; s++) {
        const q4fc_chain_step& st = steps[s];
        const int64_t Kg = (st.K + G - 1) / G;
        if (st.K <= 0 || st.K % 8 != 0 || st.njobs <= 0 || jcur + st.njobs > njobs || !st.x) {
            set_error("fc_chain: step %d: K=%lld must be a positive multiple of 8, njobs=%d >= 1 inside the %d jobs given, x non-null",
                      s, (long long)st.K, st.njobs, njobs);
            return Q4FC_EINVAL;
        }
        if (st.transform < Q4FC_CHAIN_PLAIN || st.transform > Q4FC_CHAIN_SILU_MUL ||
            (st.transform != Q4FC_CHAIN_PLAIN && !st.aux)) {
            set_error("fc_chain: step %d: transform %d needs its second operand", s, st.transform);
            return Q4FC_EINVAL;
        }
        if (st.ldx < st.K || st.ldx % 4 != 0 || (reinterpret_cast<uintptr_t>(st.x) & 15) ||
            (reinterpret_cast<uintptr_t>(st.aux) & 15)) {
            set_error("fc_chain: step %d: x and its second operand need 16-byte alignment and ldx %% 4 == 0, ldx >= K", s);
            return Q4FC_EALIGN;
        }
        if (Kg >= (1 << 20) || st.ldx >= 0x7fffffffLL) {
            set_error("fc_chain: step %d: K=%lld / ldx=%lld beyond the limit", s, (long long)st.K, (long long)st.ldx);
            return Q4FC_ELIMIT;
        }
        ChainStepDev& d = hs[(size_t)s];
        d.x = st.x, d.aux = st.aux, d.ldx = (int)st.ldx, d.K = (int)st.K, d.eps = st.eps, d.transform = st.transform;
        d.Kg = (int)Kg, d.job0 = jcur, d.pad = 0;
        d.rot = (int)(((int64_t)s * rot_step) % di->sm_count);
        int64_t stripes = 0;
        for (int k = 0; k < st.njobs; k++, jcur++) {
            const q4fc_fc_job& j = jobs[jcur];
            if (!j.wq || !j.y || j.N <= 0 || j.Ng <= 0 || j.N > j.Ng * 32 || j.ldy < j.N) {
                set_error("fc_chain: job %d: null pointer, N=%lld not covered by Ng=%lld, or ldy < N", jcur, (long long)j.N,
                          (long long)j.Ng);
                return Q4FC_EINVAL;
            }
            if (reinterpret_cast<uintptr_t>(j.wq) & 15) {
                set_error("fc_chain: job %d: packed weights need 16-byte alignment", jcur);
                return Q4FC_EALIGN;
            }
            if (static_cast<const void*>(j.y) == static_cast<const void*>(st.x) ||
                static_cast<const void*>(j.y) == static_cast<const void*>(st.aux)) {
                set_error("fc_chain: job %d writes the input of its own step", jcur);
                return Q4FC_EINVAL;
            }
            stripes += (j.N + 31) / 32;  // stripes beyond N hold no output
            if (stripes * Kg >= 0x7fffffffLL || j.ldy >= 0x7fffffffLL || j.ld_addend >= 0x7fffffffLL) {
                set_error("fc_chain: step %d exceeds 2^31 blocks", s);
                return Q4FC_ELIMIT;
            }
            ChainJobDev& e = hj[(size_t)jcur];
            e.wq = static_cast<const uint8_t*>(j.wq), e.y = j.y, e.addend = j.addend;
            e.N = (int)j.N, e.ldy = (int)j.ldy, e.addend_ld = (int)j.ld_addend, e.s_end = (int)stripes;
        }
        d.stripes = (int)stripes;
        d.units = (int)stripes * rows;
        if (d.Kg > kg_max) kg_max = d.Kg;
    }
    if (jcur != njobs) {
        set_error("fc_chain: the steps use %d of the %d jobs given", jcur, njobs);
        return Q4FC_EINVAL;
    }
    ChainHandle* h = new ChainHandle();
    ChainParams& p = h->p;
    p.nsteps = nsteps, p.rows = rows, p.rows_p = (rows + 1) / 2 * 2;
    p.kg_max = kg_max;
    p.code_stride = (kg_max * G + 127) / 128 * 128 + 32;  // rows 32 B apart modulo 128: conflict-free operand loads
    p.slot_bytes = SB * BS;
    const size_t table_bytes = sizeof(ChainStepDev) * (size_t)nsteps + sizeof(ChainJobDev) * (size_t)njobs;
    if (table_bytes > kChainTableMax) {
        set_error("fc_chain: %d steps and %d jobs need %zu bytes of tables, more than the %zu a chain may have: cut it in two",
                  nsteps, njobs, table_bytes, kChainTableMax);
        delete h;
        return Q4FC_ELIMIT;
    }
    p.table_bytes = (int)table_bytes;
    p.part_off = (int)align_up(512 + table_bytes, 128);
    size_t fixed = (size_t)p.part_off + (size_t)kCPartBufs * kCW * p.rows_p * 32 * 4 + (size_t)kg_max * 64 + (size_t)rows * p.code_stride;
    fixed = align_up(fixed, 128);
    int64_t depth = ((int64_t)di->max_smem_optin - (int64_t)fixed) / p.slot_bytes;
    if (depth > kCRingMax) depth = kCRingMax;
    if (depth < 2) {
        set_error("fc_chain: rows=%d K=%d leave no room for the weight ring in %d bytes of shared memory", rows, kg_max * G,
                  di->max_smem_optin);
        delete h;
        return Q4FC_ELIMIT;
    }
    p.depth = (int)depth, p.ring_off = (int)fixed;
    h->smem = fixed + (size_t)depth * p.slot_bytes;
    if (qtype == 1 && G == 32) h->fn = chain_fn_for_rows<32, 1>(rows);
    else if (qtype == 1) h->fn = chain_fn_for_rows<128, 1>(rows);
    else if (G == 32) h->fn = chain_fn_for_rows<32, 0>(rows);
    else h->fn = chain_fn_for_rows<128, 0>(rows);
    cudaError_t e = cudaGetDevice(&h->device);
    if (e == cudaSuccess) {
        std::lock_guard<std::mutex> lk(g_chain_mutex);
        e = cudaFuncSetAttribute(h->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin);
    }
    int per_sm = 0;
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, h->fn, kCThreads, h->smem);
    if (e != cudaSuccess || per_sm < 1) {
        delete h;
        if (e != cudaSuccess) return cuda_fail(e, "fc_chain: kernel set-up");
        set_error("fc_chain: the kernel does not fit an SM with %zu bytes of shared memory", fixed + (size_t)depth * p.slot_bytes);
        return Q4FC_ELIMIT;
    }
    h->grid = di->sm_count;  // one CTA per SM, all resident (cooperative launch)
    const size_t steps_bytes = sizeof(ChainStepDev) * (size_t)nsteps;  // the jobs follow directly: one copy into shared memory
    const size_t jobs_bytes = align_up(steps_bytes + sizeof(ChainJobDev) * (size_t)njobs, 256) - steps_bytes;
    const size_t sync_bytes = 768 + 128 * (size_t)nsteps;  // launches, leavers, status, then the steps' counters
    const size_t total = steps_bytes + jobs_bytes + sync_bytes;
    e = cudaMalloc(&h->dev, total);
    if (e != cudaSuccess) {
        delete h;
        return cuda_fail(e, "fc_chain: cudaMalloc of the step tables");
    }
    uint8_t* base = static_cast<uint8_t*>(h->dev);
    e = cudaMemset(base + steps_bytes + jobs_bytes, 0, sync_bytes);
    if (e == cudaSuccess) e = cudaMemcpy(base, hs.data(), sizeof(ChainStepDev) * (size_t)nsteps, cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
        e = cudaMemcpy(base + steps_bytes, hj.data(), sizeof(ChainJobDev) * (size_t)njobs, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(h->dev);
        delete h;
        return cuda_fail(e, "fc_chain: upload of the step tables");
    }
    p.steps = reinterpret_cast<const ChainStepDev*>(base);
    p.jobs = reinterpret_cast<const ChainJobDev*>(base + steps_bytes);
    // every word that is polled or counted on sits on a line of its own
    p.launches = reinterpret_cast<unsigned*>(base + steps_bytes + jobs_bytes);
    p.leavers = reinterpret_cast<unsigned*>(base + steps_bytes + jobs_bytes + 256);
    p.status = reinterpret_cast<int*>(base + steps_bytes + jobs_bytes + 512);
    p.arrivals = reinterpret_cast<unsigned*>(base + steps_bytes + jobs_bytes + 768);
    h->sync_bytes = sync_bytes;
    *out = h;
    return Q4FC_OK;
}

int chain_run(void* chain, cudaStream_t s) {
    ChainHandle* h = static_cast<ChainHandle*>(chain);
    int dev = -1;
    Q4FC_CUDA_OK(cudaGetDevice(&dev));
    if (dev != h->device) {
        set_error("fc_chain: made on device %d, run on device %d", h->device, dev);
        return Q4FC_EINVAL;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)h->grid);
    cfg.blockDim = dim3(kCThreads);
    cfg.dynamicSmemBytes = h->smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // every CTA resident: the grid barrier needs them all
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    void* args[] = {&h->p};
    Q4FC_CUDA_OK(cudaLaunchKernelExC(&cfg, h->fn, args));
    return Q4FC_OK;
}

int chain_check(void* chain, cudaStream_t s) {
    ChainHandle* h = static_cast<ChainHandle*>(chain);
    int status = 0;
    Q4FC_CUDA_OK(cudaMemcpyAsync(&status, h->p.status, sizeof(int), cudaMemcpyDeviceToHost, s));
    Q4FC_CUDA_OK(cudaStreamSynchronize(s));
    if (status != 0) {
        // the counters are left mid-count by a launch that gave up: clear them with the status
        Q4FC_CUDA_OK(cudaMemsetAsync(h->p.launches, 0, h->sync_bytes, s));
        Q4FC_CUDA_OK(cudaStreamSynchronize(s));
        set_error("fc_chain: device status word = 0x%x (a bounded wait ran out)", status);
        return Q4FC_EDEVICE;
    }
    return Q4FC_OK;
}

int chain_destroy(void* chain) {
    ChainHandle* h = static_cast<ChainHandle*>(chain);
    if (!h) return Q4FC_OK;
    const cudaError_t e = cudaFree(h->dev);
    delete h;
    if (e != cudaSuccess) return cuda_fail(e, "fc_chain: cudaFree");
    return Q4FC_OK;
}

}  // namespace q4fc
