// Decode FC (rows <= 8): the kernel behind q4fc_fc_decode / _q8 / _add / _multi, and with TP = true behind
// q4fc_fc_decode_tp.  Included by fc_decode_ring.cu (TP = false) and fc_decode_ring_tp.cu (TP = true): two
// translation units, so that the multi-GPU code paths cost the single-GPU instantiations nothing.
// Reference arithmetic: fc_Q4A, ops/op_fc.hpp:286-426 (shared pieces in decode_math.cuh).
//
// Work.  One CTA per SM.  A launch carries up to 16 "jobs" (weight tensors), each multiplying one of up to 16
// inputs: the q/k/v projections of one activation, gate and up, or any batch of independent FCs.  The stripes
// (32 output columns, Kg blocks of BS contiguous bytes each) of all jobs form one index space, cut into
// contiguous ranges of about equal bytes, one per CTA, so a whole batch streams as one launch with no kernel
// boundary in it.  When a single input has fewer stripes than half the SMs, a thread-block cluster of cs CTAs
// shares a stripe range and CTA rank j takes the K slice [j*Kg/cs, (j+1)*Kg/cs) of each of them.
//
// Streaming.  Warp 8 is the producer: one thread walks the CTA's byte stream and issues 1-D bulk copies
// (cp.async.bulk, global -> shared, completion counted on an mbarrier; this GPU's own memory, no multicast) of
// up to SB blocks each into a ring of `depth` slots, as far ahead as the ring allows -- on B200 that is up to
// ~190 KB per SM in flight with no register cost, and for most Llama-7B shapes the CTA's whole share.  The
// first ring-full is issued before the programmatic-dependent-launch wait: weights never depend on the
// preceding kernel, so they stream while that kernel drains and while this one quantizes its activations.
// Warps 0-15 consume: every warp takes block(s) `warp` of each slot from shared memory into registers, frees
// the slot with one mbarrier arrival per warp, feeds mma.sync.m16n8k32 (u8 x s8 -> s32, exact) and scales per
// K group in fp32.
//
// Reduction.  At the end of a stripe the warps' partial sums meet in shared memory (four buffers, handed over
// with mbarriers so that nobody waits for the slowest warp) and one warp per row -- the duty moves round the
// warps -- adds them in warp order: fixed order, no atomics, no global scratch.  With cs > 1 the CTA's sum goes over distributed shared memory into the inbox of the stripe's owner
// (rank = stripe mod cs), which adds the cs contributions in rank order after one cluster barrier.
//
// Activations.  Either quantized here (one input; a warp takes 128 consecutive k of up to four rows; codes and
// scales bit-equal to FC_dynamic_quantize_x, ops/op_fc.hpp:246-268, group sums tree-ordered; without a K split
// every CTA needs all of them, so clusters of four CTAs split that work and store the codes into one another's
// shared memory), or -- PREQ -- fetched, already quantized, with bulk copies (q4fc_quant_x_q8 /
// q4fc_rmsnorm_quant / q4fc_silu_mul_quant made them); a CTA whose range crosses from one input to the next
// fetches the next input's codes when it gets there, while its weight ring keeps filling.
//
// Every wait is bounded (one second by %globaltimer): when it runs out the status word is set, the CTA's
// other waits end at once, all roles run to the end of their loops (no barrier is left waiting for anyone)
// and the kernel returns after a short pause for copies still in flight.
#pragma once
#include <cooperative_groups.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "decode_math.cuh"
#include "ring_ptx.cuh"

namespace cg = cooperative_groups;

namespace q4fc {
namespace {

constexpr int kRW = 16;  // consumer warps
constexpr int kRThreads = (kRW + 1) * 32;
constexpr int kRingMax = 10;    // most slots a ring can have
constexpr int kPartBufs = 4;    // buffers in which the warps' partial sums of successive stripes meet
constexpr int kMaxJobs = 16;    // weight tensors per launch
constexpr int kMaxInputs = 16;  // distinct activation tensors per launch
constexpr int kMaxTpJobs = 4;   // weight tensors per launch in the multi-GPU form
constexpr int kMaxUnits = 160;  // work units (CTAs, or clusters) per launch: bounds the table of first stripes
constexpr int kShare = 4;       // CTAs that share the quantization of the activations (cs == 1)
constexpr int kMaxOwned = 16;   // stripes per cluster when cs > 1 (bounds the inbox)

struct RingJobDev {
    const uint8_t* wq;
    float* y;
    const float* addend;  // optional: y = fc(x) + addend; addend_ld = 0 broadcasts one row (a bias)
    int64_t N, ldy, addend_ld;
    int s_end;  // one past this job's last stripe in the launch's common stripe index space
    int input;  // which activation tensor it multiplies
};
struct RingInputDev {
    const int8_t* xq;  // PREQ: codes [rows][xq_stride], scales and group sums [Kg][16]
    const float* xsc;
    int64_t xq_stride, K;
    int rows, Kg;
};
struct RingParams {
    const float* x;  // fused quantizer (one input): fp32 [rows][ldx]; TP with x_stamped: stamped words [rows][ldx]
    int64_t ldx;
    int njobs, ninputs;
    RingJobDev job[kMaxJobs];
    RingInputDev in[kMaxInputs];
    int unit_s0[kMaxUnits + 1];  // first stripe of work unit u; [nc] = number of stripes
    int rows_max, rows_p;        // most rows of any input; that rounded up to even
    int cs, log2cs, nc;          // K split: CTAs per cluster (power of two); work units (clusters, or CTAs when cs == 1)
    int bq;                      // cs == 1, fused quantizer: CTAs (a power of two) that share the quantization
    int kq, kr;                  // cs > 1 (one input): K groups per rank: kq, the first kr ranks one more
    int kc_max;                  // most K groups a CTA's slice can have
    int code_stride;             // bytes between code rows in shared memory
    int depth, slot_bytes, ring_off;
    int inbox_stripes;  // stripes a CTA can own (cs > 1)
    int x_vec_ok;
    int* status;  // set non-zero when a bounded wait ran out
    // N-split over several GPUs (TP): outputs leave as 8-byte stamped words (fp32 value, low 32 bits of the step
    // counter) stored into every rank's buffer; a 64-bit store is indivisible, so a reader that finds the
    // current stamp has the value too
    int world, x_stamped;
    int64_t col_off[kMaxTpJobs];
    unsigned long long* y_peer[kMaxTpJobs][8];
    const unsigned long long* epoch;
};

__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__device__ __forceinline__ unsigned long long ld_stamped(const unsigned long long* a) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(a) : "memory");
    return w;
}
__device__ __forceinline__ void st_stamped(unsigned long long* a, float v, uint32_t stamp) {
    const unsigned long long w = ((unsigned long long)stamp << 32) | __float_as_uint(v);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(a), "l"(w) : "memory");
}

template <int G, int QTYPE>
struct RingShape {
    static constexpr int BS = block_bytes(QTYPE, G);
    static constexpr int SETS = G / 32;
    static constexpr int NBLK = (G == 32) ? 4 : 1;  // consecutive blocks a warp takes from a slot
    static constexpr int SB = kRW * NBLK;           // blocks per slot
    static constexpr int SLOT = SB * BS;
};

// ---- the consumer warps quantize this CTA's K slice of the rows (ops/op_fc.hpp:246-268) ------------------
template <int G, int ROWS, bool SIGNED, bool TP>
__device__ __forceinline__ void quantize_slice(const RingParams& p, int warp, int lane, int k0, int Kc, uint8_t* codes,
                                               float* sc, uint32_t stamp, int jq, int bq, cg::cluster_group& cluster, int rows,
                                               int64_t K) {
    constexpr int SEG = G / 4;    // lanes per group
    constexpr int GPC = 128 / G;  // groups per 128-k chunk
    constexpr int RI = ROWS > 4 ? 4 : ROWS;  // rows a warp takes at a time: 8 rows are two work items per chunk
    constexpr int RGRP = ROWS / RI;
    const int Ls = Kc * G;  // slice length per row
    const int64_t kbase = (int64_t)k0 * G;
    const int chunks = (Ls + 127) >> 7;
    // bq CTAs of a cluster that all need the same slice share the work: item i goes to CTA (i / kRW) mod bq,
    // which stores the result into every sharer's shared memory (its own included)
    for (int item = jq * kRW + warp; item < chunks * RGRP; item += bq * kRW) {
        const int ch = item / RGRP, m0 = (item - ch * RGRP) * RI;
        const int e = ch * 128 + lane * 4;  // element inside the slice
        const int64_t k = kbase + e;
        const int kbl = ch * GPC + lane / SEG;
        const bool exists = kbl < Kc;
        const int len = exists ? (int)min((int64_t)G, K - (kbase + (int64_t)kbl * G)) : 0;
        const bool vec = p.x_vec_ok && (e < Ls) && (k + 4 <= K);
        float v[RI][4];
        bool late = false;
#pragma unroll
        for (int mm = 0; mm < RI; mm++) {
            const int m = m0 + mm;
            v[mm][0] = v[mm][1] = v[mm][2] = v[mm][3] = 0.0f;
            if (TP && m < rows && e < Ls && p.x_stamped) {
                // first try; words whose stamp is not this step's are re-read below
                const unsigned long long* src = reinterpret_cast<const unsigned long long*>(p.x) + m * p.ldx + k;
#pragma unroll
                for (int jj = 0; jj < 4; jj++)
                    if (k + jj < K) {
                        const unsigned long long w = ld_stamped(src + jj);
                        v[mm][jj] = __uint_as_float((uint32_t)w);
                        late |= (uint32_t)(w >> 32) != stamp;
                    }
            } else if (m < rows && e < Ls) {
                const float* src = p.x + m * p.ldx + k;
                if (vec) {
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(src));
                    v[mm][0] = a.x, v[mm][1] = a.y, v[mm][2] = a.z, v[mm][3] = a.w;
                } else {
#pragma unroll
                    for (int jj = 0; jj < 4; jj++)
                        if (k + jj < K) v[mm][jj] = __ldcg(src + jj);
                }
            }
        }
        if (TP && p.x_stamped) {
            if (late) {
                // some producer has not delivered yet: poll this lane's words, within the time limit
                const unsigned long long t0 = globaltimer_ns();
                for (unsigned it = 1; late; it++) {
                    late = false;
                    for (int mm = 0; mm < RI; mm++) {
                        const int m = m0 + mm;
                        if (m >= rows) break;
                        const unsigned long long* src = reinterpret_cast<const unsigned long long*>(p.x) + m * p.ldx + k;
                        for (int jj = 0; jj < 4; jj++)
                            if (k + jj < K) {
                                const unsigned long long w = ld_stamped(src + jj);
                                v[mm][jj] = __uint_as_float((uint32_t)w);
                                late |= (uint32_t)(w >> 32) != stamp;
                            }
                    }
                    if (late && (it & 63) == 0) {
                        // once the status word is set, waits end at once: a lost rank costs one limit
                        if (*reinterpret_cast<volatile int*>(p.status) != 0) break;
                        if (globaltimer_ns() - t0 > kWaitLimitNs) {
                            atomicCAS(p.status, 0, 0x54505754);  // 'TPWT': carry on with what is there
                            break;
                        }
                    }
                }
            }
            __syncwarp();
        }
        uint32_t packed[RI];
        float d[RI], aux[RI];
        q8_quantize_rows<G, RI, SIGNED>(v, lane, len, packed, d, aux);
        if (exists) {
            for (int dst = 0; dst < bq; dst++) {
                uint8_t* cd = bq > 1 ? cluster.map_shared_rank(codes, dst) : codes;
                float* sd = bq > 1 ? cluster.map_shared_rank(sc, dst) : sc;
#pragma unroll
                for (int mm = 0; mm < RI; mm++) {
                    const int m = m0 + mm;
                    if (m < rows) {
                        *reinterpret_cast<uint32_t*>(cd + m * p.code_stride + e) = packed[mm];
                        if (lane % SEG == 0) *reinterpret_cast<float2*>(sd + kbl * 16 + m * 2) = make_float2(d[mm], aux[mm]);
                    }
                }
            }
        }
    }
}

template <int G, int QTYPE, bool SIGNED, int ROWS, bool TP, bool PREQ>
__global__ void __launch_bounds__(kRThreads, 1) fc_decode_ring_kernel(const __grid_constant__ RingParams p) {
    using S = RingShape<G, QTYPE>;
    constexpr int BS = S::BS;
    constexpr int SETS = S::SETS;
    constexpr int NBLK = S::NBLK;
    constexpr int SB = S::SB;

    extern __shared__ __align__(128) uint8_t smem[];
    // [0,512): mbarriers full[kRingMax], empty[kRingMax], xbar; failure flag at 192; pfull[kPartBufs] at 256,
    // pfree[kPartBufs] at 320; then part [kPartBufs][kRW][rows_p*32] f32 | inbox [inbox_stripes][cs][rows_p*32] f32 (cs > 1) | sc [kc_max][16] f32
    //      | codes [rows_max][code_stride] | ring [depth][slot_bytes]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int cs = p.cs, bq = p.bq;
    const int j = (int)(blockIdx.x & (cs - 1));   // K-split rank in the cluster (clusters are consecutive CTAs)
    const int jq = (int)(blockIdx.x & (bq - 1));  // rank among the CTAs that share the quantization
    const int unit = (int)(blockIdx.x >> p.log2cs);  // work unit: the cluster, or with cs == 1 the CTA
    const int s0 = p.unit_s0[unit];
    const int r = p.unit_s0[unit + 1] - s0;
    const int slot_f = p.rows_p * 32;

    const uint32_t bar0 = smem_u32(smem);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kRingMax + s); };
    const uint32_t xbar = bar0 + 8u * (2 * kRingMax);
    auto pfull_bar = [&](int b) { return bar0 + 256u + 8u * b; };
    auto pfree_bar = [&](int b) { return bar0 + 320u + 8u * b; };
    volatile int* fail = reinterpret_cast<volatile int*>(smem + 192);
    float* part = reinterpret_cast<float*>(smem + 512);
    float* inbox = part + kPartBufs * kRW * slot_f;
    float* sc = inbox + (cs > 1 ? p.inbox_stripes * cs * slot_f : 0);
    uint8_t* codes = reinterpret_cast<uint8_t*>(sc + p.kc_max * 16);
    uint8_t* ring = smem + p.ring_off;
    const int depth = p.depth;

    cg::cluster_group cluster = cg::this_cluster();

    if (threadIdx.x == kRW * 32) {
        for (int i = 0; i < depth; i++) {
            mbar_init(full_bar(i), 1);
            mbar_init(empty_bar(i), kRW);
        }
        mbar_init(xbar, 1);
        for (int i = 0; i < kPartBufs; i++) {
            mbar_init(pfull_bar(i), kRW);
            mbar_init(pfree_bar(i), p.rows_max);
        }
        *fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    pdl_launch_dependents();
    // "this CTA runs": nobody may store into a CTA's shared memory before that CTA has started
    if (cs > 1 || bq > 1) cluster_arrive_release();

    // what this CTA has to do for global stripe sg: job, index inside the job, input, K slice, first byte
    struct Stripe {
        int jb, ls, in, Kc, k0;
        const uint8_t* base;
    };
    auto describe = [&](int sg) {
        Stripe d;
        d.jb = 0;
        while (d.jb + 1 < p.njobs && sg >= p.job[d.jb].s_end) d.jb++;
        d.ls = sg - (d.jb ? p.job[d.jb - 1].s_end : 0);
        d.in = p.job[d.jb].input;
        const int Kg = p.in[d.in].Kg;
        d.k0 = cs > 1 ? j * p.kq + min(j, p.kr) : 0;
        d.Kc = cs > 1 ? p.kq + (j < p.kr ? 1 : 0) : Kg;  // >= 1: the launcher keeps cs <= Kg
        d.base = p.job[d.jb].wq + ((int64_t)d.ls * Kg + d.k0) * BS;
        return d;
    };
    // bulk copies of one input's quantized activations (this CTA's K slice) into shared memory
    auto fetch_codes = [&](int in, int k0, int Kc) {
        const RingInputDev& I = p.in[in];
        const uint32_t row_bytes = (uint32_t)(Kc * G);
        mbar_expect_tx(xbar, row_bytes * I.rows + (uint32_t)Kc * 64u);
        for (int m = 0; m < I.rows; m++)
            bulk_g2s(smem_u32(codes + m * p.code_stride), I.xq + (int64_t)m * I.xq_stride + (int64_t)k0 * G, row_bytes,
                     xbar);
        bulk_g2s(smem_u32(sc), I.xsc + (int64_t)k0 * 16, (uint32_t)Kc * 64u, xbar);
    };

    // ---- producer state (used by one thread): next slot = blocks [p_kb, p_kb + SB) of stripe p_li
    int p_li = 0, p_kb = 0, p_s = 0;
    Stripe p_d = {};
    if (r > 0) p_d = describe(s0);
    auto issue_slot = [&]() {
        const int nblk = min(SB, p_d.Kc - p_kb);
        const uint32_t bytes = (uint32_t)nblk * BS;
        mbar_expect_tx(full_bar(p_s), bytes);
        bulk_g2s(smem_u32(ring + (size_t)p_s * p.slot_bytes), p_d.base + (int64_t)p_kb * BS, bytes, full_bar(p_s));
        p_kb += SB;
        if (p_kb >= p_d.Kc) {
            p_kb = 0, p_li++;
            if (p_li < r) p_d = describe(s0 + p_li);
        }
        if (++p_s == depth) p_s = 0;
    };

    uint32_t stamp = 0;
    int p_filled = 0;
    if (warp == kRW) {
        if (lane == 0) {
            // weights do not depend on the preceding kernel: fill the ring now
            while (p_filled < depth && p_li < r) issue_slot(), p_filled++;
            if constexpr (PREQ) {
                pdl_wait_prior_grid();
                if (r > 0) {
                    const Stripe d = describe(s0);
                    fetch_codes(d.in, d.k0, d.Kc);
                }
            }
        }
        __syncwarp();
        if (bq > 1) cluster_wait_acquire();
    } else {
        pdl_wait_prior_grid();
        if constexpr (TP) stamp = (uint32_t)*reinterpret_cast<const volatile unsigned long long*>(p.epoch);
        // the sharers store into one another's shared memory: every one of them must be running first
        if (bq > 1) cluster_wait_acquire();
        if constexpr (!PREQ) {
            // one input: every stripe of the launch has the same K slice
            const int Kg = p.in[0].Kg;
            const int k0 = cs > 1 ? j * p.kq + min(j, p.kr) : 0;
            const int Kc = cs > 1 ? p.kq + (j < p.kr ? 1 : 0) : Kg;
            quantize_slice<G, ROWS, SIGNED, TP>(p, warp, lane, k0, Kc, codes, sc, stamp, jq, bq, cluster, p.in[0].rows,
                                                p.in[0].K);
        }
    }
    __syncwarp();
    if (bq > 1) {
        // codes and scales have been stored by all sharers (and this CTA's barriers are initialised)
        cluster_arrive_release();
        cluster_wait_acquire();
    } else {
        __syncthreads();  // barriers initialised; codes and scales of the slice written (fused quantizer)
        if (cs > 1) cluster_wait_acquire();  // every CTA of the cluster runs: pushes are allowed
    }

    // the finished sum of (stripe, row m, column lane) leaves the CTA
    auto final_store = [&](const Stripe& d, int m, float sum) {
        const RingJobDev& J = p.job[d.jb];
        const int64_t n = (int64_t)d.ls * 32 + lane;
        if (n < J.N) {
            if (J.addend != nullptr) sum = __fadd_rn(sum, J.addend[m * J.addend_ld + n]);
            if constexpr (!TP) {
                J.y[m * J.ldy + n] = sum;
            } else {
                for (int rk = 0; rk < p.world; rk++)
                    st_stamped(p.y_peer[d.jb][rk] + m * J.ldy + p.col_off[d.jb] + n, sum, stamp);
            }
        }
    };

    if (warp == kRW) {
        if (lane == 0) {
            // refill: a slot is reused once all consumer warps have taken their blocks out of it
            uint32_t eph = 0;  // parity of the empty barrier's completion to wait for
            int wrapped = 0;
            while (p_li < r) {
                mbar_wait(empty_bar(p_s), eph, fail, p.status, 0x52454D50);  // 'REMP'
                issue_slot();
                if (++wrapped == depth) wrapped = 0, eph ^= 1;
            }
        }
    } else {
        uint32_t xph = 0;  // parity of the activation fetch to wait for
        int cur_in = -1;
        if constexpr (PREQ) {
            if (r > 0) {
                mbar_wait(xbar, xph, fail, p.status, 0x52584251);  // 'RXBQ'
                xph ^= 1;
                cur_in = describe(s0).in;
            }
        }
        const uint8_t* my_codes = codes + g * p.code_stride + 8 * t;
        int cs_ = 0;       // consumer ring position
        uint32_t fph = 0;  // parity of the full barrier's completion to wait for
        for (int li = 0; li < r; li++) {
            const Stripe d = describe(s0 + li);
            if constexpr (PREQ) {
                if (d.in != cur_in) {
                    // the range crosses into another input: when every warp is done with the old codes, fetch
                    // the new ones (the weight ring keeps filling meanwhile)
                    asm volatile("bar.sync 1, %0;" ::"n"(kRW * 32) : "memory");
                    if (threadIdx.x == 0) fetch_codes(d.in, d.k0, d.Kc);
                    mbar_wait(xbar, xph, fail, p.status, 0x52584251);
                    xph ^= 1;
                    cur_in = d.in;
                }
            }
            const int rows = p.in[d.in].rows;
            const bool row_live = g < rows;
            float acc[4][2];
#pragma unroll
            for (int i = 0; i < 4; i++) acc[i][0] = acc[i][1] = 0.0f;
            for (int kb0 = 0; kb0 < d.Kc; kb0 += SB) {
                mbar_wait(full_bar(cs_), fph, fail, p.status, 0x5246554C);  // 'RFUL'
                const int nblk = min(SB, d.Kc - kb0);
                const uint8_t* slot = ring + (size_t)cs_ * p.slot_bytes;
                // fetch this warp's block(s) into registers, hand the slot back, then compute: the slot is held
                // for the time of a few loads, so nearly the whole ring is in flight at any moment
                uint4 q[NBLK][SETS];
                uint2 wd[NBLK], wm[NBLK];
#pragma unroll
                for (int i = 0; i < NBLK; i++) {
                    const int b = warp * NBLK + i;
                    wd[i] = wm[i] = make_uint2(0u, 0u);
                    if (b < nblk) {
                        const uint8_t* blk = slot + b * BS;
                        // Block rows are 128 bytes apart, so the four lanes (g, 0..3) of an MMA row meet in the
                        // same banks: a 128-bit load per lane costs 16 wavefronts instead of 4.  Two 64-bit loads
                        // whose halves swap with the parity of t cost 8 and four selects.
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
                if (lane == 0) mbar_arrive(empty_bar(cs_));  // release: ordered behind this warp's loads
#pragma unroll
                for (int i = 0; i < NBLK; i++) {
                    const int b = warp * NBLK + i;
                    if (b < nblk) {
                        const int ck = kb0 + b;
                        // (one activation row: only row 2t of the lane's two rows is converted and scaled)
                        block_accumulate<G, QTYPE, SIGNED, (ROWS == 1 ? 1 : 2)>(q[i], wd[i], wm[i], my_codes + ck * G,
                                                                                row_live, sc + ck * 16, t, acc);
                    }
                }
                if (++cs_ == depth) cs_ = 0, fph ^= 1;
            }
            // ---- the stripe's slice is done: the warps' partial sums meet in shared memory.
            // kPartBufs buffers take turns.  Writers do not wait for one another: a warp stores its sums, arrives
            // on the buffer's "full" barrier and goes on to the next stripe.  Row m of stripe li is added, in warp
            // order, by warp (li * rows_max + m) mod kRW -- the adding moves round the warps, so no warp is the
            // slow one -- which then arrives on the "free" barrier; a writer passes that barrier before it touches
            // the buffer again kPartBufs stripes later.
            const int buf = li % kPartBufs;
            const uint32_t use = (uint32_t)(li / kPartBufs);
            if (use > 0) mbar_wait(pfree_bar(buf), (use - 1) & 1, fail, p.status, 0x52504652);  // 'RPFR'
            float* pw = part + (buf * kRW + warp) * slot_f;
#pragma unroll
            for (int mi = 0; mi < 2; mi++)
                if ((2 * t + mi) < p.rows_p)
                    *reinterpret_cast<float4*>(pw + (2 * t + mi) * 32 + g * 4) =
                        make_float4(acc[0][mi], acc[1][mi], acc[2][mi], acc[3][mi]);
            __syncwarp();
            if (lane == 0) mbar_arrive(pfull_bar(buf));
            const int m = ((warp - li * p.rows_max) % kRW + kRW) % kRW;  // the row this warp adds, if any
            if (m < p.rows_max) {
                mbar_wait(pfull_bar(buf), use & 1, fail, p.status, 0x52504655);  // 'RPFU'
                const float* src = part + buf * kRW * slot_f + m * 32 + lane;
                float sum = 0.0f;
                if (m < rows) {
                    sum = src[0];
#pragma unroll
                    for (int w = 1; w < kRW; w++) sum += src[w * slot_f];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(pfree_bar(buf));
                if (m < rows) {
                    if (cs > 1) {
                        float* dst = inbox + (((li >> p.log2cs) << p.log2cs) + j) * slot_f + m * 32 + lane;
                        const int owner = li & (cs - 1);
                        if (owner != j) dst = cluster.map_shared_rank(dst, owner);
                        *dst = sum;
                    } else {
                        final_store(d, m, sum);
                    }
                }
            }
        }
    }

    __syncwarp();
    if (cs > 1) {
        // every slice sum has been pushed: the owner adds its stripes' cs contributions in rank order
        cluster_arrive_release();
        cluster_wait_acquire();
        if (warp < p.rows_max) {  // consumer warp m: row m (cs > 1 has one input: rows_max is its row count)
            for (int li = j; li < r; li += cs) {
                const float* src = inbox + ((li >> p.log2cs) << p.log2cs) * slot_f + warp * 32 + lane;
                float sum = src[0];
                for (int q = 1; q < cs; q++) sum += src[q * slot_f];
                final_store(describe(s0 + li), warp, sum);
            }
        }
        // no CTA touches another CTA's shared memory after the barrier above, so exiting is safe
    }
    if (*fail != 0) {
        // a wait ran out: give bulk copies that may still be in flight time to land before the shared memory
        // is handed to another CTA
        for (int i = 0; i < 64; i++) __nanosleep(32000);
    }
}

// one launchable instantiation: its function pointer plus lazily set attributes (guarded by g_setup_mutex)
struct RingVariant {
    const void* fn;
    bool attr_done[64];
    int max_clusters[64][4];  // [device][log2 cs], 0 = not queried yet
};
std::mutex g_setup_mutex;

template <int G, int QTYPE, bool SIGNED, int ROWS, bool TP, bool PREQ>
RingVariant* ring_variant_of() {
    static RingVariant v = {
        reinterpret_cast<const void*>(&fc_decode_ring_kernel<G, QTYPE, SIGNED, ROWS, TP, PREQ>), {}, {}};
    return &v;
}

// The pre-quantized form has two instantiations per block type: one activation row (half the conversions and
// scalings after the MMAs), and up to eight
template <int G, int QTYPE, bool SIGNED, bool TP>
RingVariant* ring_variant_for_rows(int rows, bool preq) {
    if (preq) return rows <= 1 ? ring_variant_of<G, QTYPE, SIGNED, 1, TP, true>() : ring_variant_of<G, QTYPE, SIGNED, 8, TP, true>();
    if (rows <= 1) return ring_variant_of<G, QTYPE, SIGNED, 1, TP, false>();
    if (rows <= 2) return ring_variant_of<G, QTYPE, SIGNED, 2, TP, false>();
    if (rows <= 4) return ring_variant_of<G, QTYPE, SIGNED, 4, TP, false>();
    return ring_variant_of<G, QTYPE, SIGNED, 8, TP, false>();
}

template <bool TP>
RingVariant* ring_pick_variant(int qtype, int G, bool sgn, int rows, bool preq) {
    if (qtype == 1 && G == 32) return ring_variant_for_rows<32, 1, false, TP>(rows, preq);
    if (qtype == 1 && G == 128) return ring_variant_for_rows<128, 1, false, TP>(rows, preq);
    if (qtype == 0 && G == 32 && !sgn) return ring_variant_for_rows<32, 0, false, TP>(rows, preq);
    if (qtype == 0 && G == 128 && !sgn) return ring_variant_for_rows<128, 0, false, TP>(rows, preq);
    if (qtype == 0 && G == 32) return ring_variant_for_rows<32, 0, true, TP>(rows, preq);
    return ring_variant_for_rows<128, 0, true, TP>(rows, preq);
}

void ring_fill_launch_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int grid, int cs, size_t smem, bool pdl,
                             cudaStream_t s) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kRThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    int nattr = 0;
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = (unsigned)cs;
    attr[nattr].val.clusterDim.y = 1;
    attr[nattr].val.clusterDim.z = 1;
    nattr++;
    if (pdl) {
        attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[nattr].val.programmaticStreamSerializationAllowed = 1;
        nattr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
}

// clusters of `cl` CTAs (one CTA per SM) that can be resident at once, hardware placement included; cached
int ring_max_clusters(RingVariant* v, int dev, int cl, int log2cl, const DeviceInfo* di) {
    std::lock_guard<std::mutex> lk(g_setup_mutex);
    if (v->max_clusters[dev][log2cl] == 0) {
        if (!v->attr_done[dev]) {
            const cudaError_t e =
                cudaFuncSetAttribute(v->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin);
            if (e != cudaSuccess) {
                cuda_fail(e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
                return -1;
            }
            v->attr_done[dev] = true;
        }
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[2];
        // queried at the largest footprint a CTA can have: one CTA per SM either way
        ring_fill_launch_config(cfg, attr, cl, cl, (size_t)di->max_smem_optin, false, nullptr);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, v->fn, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = di->sm_count / cl / 2;  // conservative stand-in
            if (n < 1) n = 1;
        }
        v->max_clusters[dev][log2cl] = n;
    }
    return v->max_clusters[dev][log2cl];
}

// Above this many activation values (rows x K) a separate quantizing launch in front of the FC beats the
// quantizer inside it, which every CTA (or cluster of sharers) runs for itself.  Needs scratch: used only when
// the caller's workspace has room for it.
constexpr int64_t kPreQuantMinValues = 40 * 1024;

// one FC of a launch, as the entry points describe it
struct RingCall {
    const float* x;  // fp32 [rows][ldx], or nullptr when xq is given
    int64_t ldx;
    const void* xq;  // activations quantized beforehand (q4fc_xq_* format), or nullptr
    int rows;
    int64_t K, Kg;
    const uint8_t* wq;
    int64_t Ng, N;
    float* y;
    int64_t ldy;
    const float* addend;
    int64_t addend_ld;
};

template <bool TP>
int launch_ring_impl(const RingCall* calls, int ncalls, int qtype, int G, unsigned flags, cudaStream_t s,
                     const q4fc_tp_site* const* tp, void* ws, size_t ws_bytes) {
    const DeviceInfo* di = device_info();
    if (!di) return Q4FC_ECUDA;
    RingParams p = {};
    // ---- jobs and the inputs they read (calls with the same input pointer share one input)
    const void* in_key[kMaxInputs];
    int64_t ng_total = 0, blocks_total = 0;
    bool any_fp32 = false;
    for (int i = 0; i < ncalls; i++) {
        const RingCall& c = calls[i];
        // a tensor (or a rank's shard) without columns, or a call without rows, takes no part
        if (c.rows == 0 || c.N == 0 || c.Ng == 0) continue;
        if (p.njobs == (TP ? kMaxTpJobs : kMaxJobs)) {
            set_error("fc_decode: more than %d weight tensors in one launch", TP ? kMaxTpJobs : kMaxJobs);
            return Q4FC_ELIMIT;
        }
        const void* key = c.xq ? c.xq : static_cast<const void*>(c.x);
        int in = 0;
        while (in < p.ninputs && in_key[in] != key) in++;
        if (in == p.ninputs) {
            if (p.ninputs == kMaxInputs) {
                set_error("fc_decode: more than %d inputs in one launch", kMaxInputs);
                return Q4FC_ELIMIT;
            }
            in_key[in] = key;
            RingInputDev& I = p.in[in];
            I.rows = c.rows, I.K = c.K, I.Kg = (int)c.Kg, I.xq_stride = c.Kg * G;
            if (c.xq) {
                const uint8_t* base = static_cast<const uint8_t*>(c.xq);
                I.xq = reinterpret_cast<const int8_t*>(base);
                I.xsc = reinterpret_cast<const float*>(base + align_up((size_t)(c.rows * c.Kg * G), 256));
            } else {
                any_fp32 = true;
                p.x = c.x, p.ldx = c.ldx;
            }
            p.ninputs++;
        } else if (p.in[in].rows != c.rows || p.in[in].K != c.K) {
            set_error("fc_decode: two calls share an input pointer but not its shape");
            return Q4FC_EINVAL;
        }
        RingJobDev& J = p.job[p.njobs];
        J.wq = c.wq, J.y = c.y, J.addend = c.addend, J.N = c.N, J.ldy = c.ldy, J.addend_ld = c.addend_ld, J.input = in;
        ng_total += c.Ng;
        blocks_total += c.Ng * c.Kg;
        if (blocks_total >= 0x7fffffffLL) {
            set_error("fc_decode: %lld blocks exceed the 2^31 limit", (long long)blocks_total);
            return Q4FC_ELIMIT;
        }
        J.s_end = (int)ng_total;
        if (TP) {
            const q4fc_tp_site* t = tp[i];
            p.col_off[p.njobs] = t->col_off;
            for (int rk = 0; rk < t->world; rk++) p.y_peer[p.njobs][rk] = t->y_peer[rk];
        }
        p.njobs++;
    }
    if (p.njobs == 0) return Q4FC_OK;
    if (any_fp32 && p.ninputs > 1) {
        set_error("fc_decode: a launch over several inputs needs them quantized beforehand (q4fc_quant_x_q8)");
        return Q4FC_EINVAL;
    }
    int rows_max = 0, kg_max = 0;
    for (int i = 0; i < p.ninputs; i++) {
        if (p.in[i].rows > rows_max) rows_max = p.in[i].rows;
        if (p.in[i].Kg > kg_max) kg_max = p.in[i].Kg;
    }
    p.rows_max = rows_max, p.rows_p = (rows_max + 1) / 2 * 2;
    int* status = ws ? static_cast<int*>(ws) : ring_status_word();
    if (TP) {
        p.world = tp[0]->world, p.x_stamped = tp[0]->x_stamped, p.epoch = tp[0]->epoch;
        status = tp[0]->status;
    }
    if (!status) return Q4FC_ECUDA;
    p.status = status;
    const bool sgn = (flags & Q4FC_FLAG_NIBBLE_SIGNED) && qtype == 0;
    const bool pdl = (flags & Q4FC_FLAG_PDL) != 0;

    // ---- one fp32 input: quantize it inside the FC kernel, or in a launch of its own in front of it
    bool preq = !any_fp32, own_quant_launch = false;
    if (any_fp32) {
        const int rows = p.in[0].rows;
        const int64_t K = p.in[0].K, Kg = p.in[0].Kg;
        uint8_t* base = nullptr;
        if (TP && tp[0]->xq_scratch != nullptr && !tp[0]->x_stamped) {
            base = static_cast<uint8_t*>(tp[0]->xq_scratch);  // the caller's scratch
        } else if (!TP && ws != nullptr &&
                   ((flags & Q4FC_FLAG_PREQUANT) || (int64_t)rows * K >= kPreQuantMinValues) &&
                   ws_bytes >= decode_prequant_offset() + quant_pre_bytes(rows, K, G)) {
            base = static_cast<uint8_t*>(ws) + decode_prequant_offset();  // its fixed place in the workspace
        }
        if (base) {
            p.in[0].xq = reinterpret_cast<const int8_t*>(base);
            p.in[0].xsc = reinterpret_cast<const float*>(base + align_up((size_t)(rows * Kg * G), 256));
            preq = own_quant_launch = true;
        }
    }
    RingVariant* v = ring_pick_variant<TP>(qtype, G, sgn, rows_max, preq);
    int dev = 0;
    Q4FC_CUDA_OK(cudaGetDevice(&dev));
    if (dev >= 64) {
        set_error("fc_decode: device index %d beyond the 64 this library keeps state for", dev);
        return Q4FC_ELIMIT;
    }

    // ---- shape of the launch: K split (clusters) only when one input's stripes alone cannot fill the GPU
    const int sms = di->sm_count;
    const int BS = block_bytes(qtype, G);
    const int SB = kRW * (G == 32 ? 4 : 1);
    p.slot_bytes = SB * BS;
    int cs = 1;
    if (p.ninputs == 1)
        while (cs < 8 && cs * 2 <= kg_max && ng_total * cs * 2 <= sms) cs *= 2;
    size_t fixed = 0;
    int nc = 0;
    for (;; cs *= 2) {
        p.cs = cs;
        p.log2cs = 0;
        while ((1 << p.log2cs) < cs) p.log2cs++;
        p.kq = kg_max / cs, p.kr = kg_max % cs;
        p.kc_max = cs > 1 ? p.kq + (p.kr > 0 ? 1 : 0) : kg_max;
        p.code_stride = (p.kc_max * G + 127) / 128 * 128 + 32;  // rows 32 B apart modulo 128: conflict-free operand loads
        int nc_cap = sms / cs;
        if (cs > 1) {
            nc_cap = ring_max_clusters(v, dev, cs, p.log2cs, di);
            if (nc_cap < 0) return Q4FC_ECUDA;
        }
        if (nc_cap > kMaxUnits) nc_cap = kMaxUnits;
        // all units resident at once (one wave); with cs > 1 at most kMaxOwned stripes per cluster
        nc = (int)(ng_total < nc_cap ? ng_total : nc_cap);
        if (cs > 1) {
            const int64_t nc_lo = (ng_total + kMaxOwned - 1) / kMaxOwned;
            if (nc < nc_lo) nc = (int)(nc_lo < kMaxUnits ? nc_lo : kMaxUnits);
        }
        const int r_max = (int)((ng_total + nc - 1) / nc);
        p.inbox_stripes = cs > 1 ? (r_max + cs - 1) / cs : 0;
        const size_t slot_f = (size_t)p.rows_p * 32;
        fixed = 512 + kPartBufs * kRW * slot_f * 4 + (size_t)p.inbox_stripes * cs * slot_f * 4 + (size_t)p.kc_max * 64 +
                (size_t)rows_max * p.code_stride;
        fixed = align_up(fixed, 128);
        if (fixed + 2 * (size_t)p.slot_bytes <= (size_t)di->max_smem_optin) break;
        if (p.ninputs > 1 || cs >= 8 || cs * 2 > kg_max) {
            set_error("fc_decode: rows=%d Kg=%d needs %zu bytes of shared memory (limit %d)", rows_max, kg_max,
                      fixed + 2 * (size_t)p.slot_bytes, di->max_smem_optin);
            return Q4FC_ELIMIT;
        }
    }
    p.ring_off = (int)fixed;
    // Without a K split every CTA needs all of the quantized activations: clusters of kShare CTAs split that work
    // and store the codes into one another's shared memory, instead of each CTA repeating it.
    p.bq = 1;
    if (p.cs == 1 && !preq) {
        int bq = kShare;
        while (bq > 1 && nc < bq) bq /= 2;
        if (bq > 1) {
            int l2 = 0;
            while ((1 << l2) < bq) l2++;
            const int cap = ring_max_clusters(v, dev, bq, l2, di);
            if (cap < 0) return Q4FC_ECUDA;
            int units = nc / bq * bq;
            if (units > cap * bq) units = cap * bq;
            p.bq = bq;
            nc = units;
        }
    }
    p.nc = nc;
    // ---- stripes -> units: contiguous ranges of about equal bytes (stripes of different jobs differ in length)
    {
        int64_t done_blocks = 0;  // blocks of all stripes before the cursor
        int jb = 0;
        int64_t s = 0;  // cursor: global stripe index
        p.unit_s0[0] = 0;
        for (int u = 1; u < nc; u++) {
            const int64_t target = blocks_total * u / nc;
            // advance whole jobs, then stripes inside the job, until `target` blocks lie behind the cursor
            for (;;) {
                const int64_t kg = p.in[p.job[jb].input].Kg;
                const int64_t left = p.job[jb].s_end - s;  // stripes left in this job
                if (done_blocks + left * kg <= target && jb + 1 < p.njobs) {
                    done_blocks += left * kg, s = p.job[jb].s_end, jb++;
                    continue;
                }
                int64_t step = (target - done_blocks + kg - 1) / kg;  // round up: never behind the target
                if (step > left) step = left;
                if (step < 0) step = 0;
                done_blocks += step * kg, s += step;
                break;
            }
            p.unit_s0[u] = (int)s;
        }
        p.unit_s0[nc] = (int)ng_total;
    }
    {
        // as deep as the shared memory allows, but no deeper than the launch has slots
        int64_t want = 0;
        for (int k = 0; k < p.njobs; k++) {
            const int64_t kc = cs > 1 ? p.kc_max : p.in[p.job[k].input].Kg;
            want += (int64_t)(p.job[k].s_end - (k ? p.job[k - 1].s_end : 0)) * ((kc + SB - 1) / SB);
        }
        int64_t depth = ((int64_t)di->max_smem_optin - (int64_t)fixed) / p.slot_bytes;
        if (depth > kRingMax) depth = kRingMax;
        if (depth > want) depth = want;
        if (depth < 1) depth = 1;
        p.depth = (int)depth;
    }
    const size_t smem = fixed + (size_t)p.depth * p.slot_bytes;
    p.x_vec_ok = any_fp32 && (p.in[0].K % 4 == 0) && (p.ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 15) == 0);
    {
        std::lock_guard<std::mutex> lk(g_setup_mutex);
        if (!v->attr_done[dev]) {
            Q4FC_CUDA_OK(cudaFuncSetAttribute(v->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin));
            v->attr_done[dev] = true;
        }
    }
    if (own_quant_launch) {
        if (int rc = launch_quant_x_pre(p.x, p.in[0].rows, p.in[0].K, p.ldx, G, sgn, const_cast<int8_t*>(p.in[0].xq),
                                        const_cast<float*>(p.in[0].xsc), pdl, s))
            return rc;
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    // behind its own quantizing launch the FC always starts early: its weight copies run beside that launch
    ring_fill_launch_config(cfg, attr, p.nc * p.cs, p.cs > 1 ? p.cs : p.bq, smem, pdl || own_quant_launch, s);
    void* args[] = {const_cast<RingParams*>(&p)};
    Q4FC_CUDA_OK(cudaLaunchKernelExC(&cfg, v->fn, args));
    return Q4FC_OK;
}

}  // namespace
}  // namespace q4fc
