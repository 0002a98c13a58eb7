// Decode FC (rows <= 8): the kernel behind q4fc_fc_decode / _q8 / _add / _multi, and with TP = true behind
// q4fc_fc_decode_tp.  Included by fc_decode_ring.cu (TP = false) and fc_decode_ring_tp.cu (TP = true): two
// translation units, so that the multi-GPU code paths cost the single-GPU instantiations nothing.
// Reference arithmetic: fc_Q4A, ops/op_fc.hpp:286-426 (shared pieces in decode_math.cuh).
//
// Work.  One CTA per SM.  A CTA owns a contiguous range of stripes (32 output columns, Kg blocks of BS
// contiguous bytes each); the stripes of up to four weight tensors that share one input ("jobs": q/k/v, or
// gate/up) form one index space.  When there are fewer stripes than half the SMs, a thread-block cluster of
// cs CTAs shares a stripe range and CTA rank j takes the K slice [j*Kg/cs, (j+1)*Kg/cs) of each of them.
//
// Streaming.  Warp 8 is the producer: one thread walks the CTA's byte stream and issues 1-D bulk copies
// (cp.async.bulk, global -> shared, completion counted on an mbarrier; this GPU's own memory, no multicast) of
// up to SB blocks each into a ring of `depth` slots, as far ahead as the ring allows -- on B200 that is up to
// ~190 KB per SM in flight with no register cost, and for most Llama-7B shapes the CTA's whole share.  The
// first ring-full is issued before the programmatic-dependent-launch wait: weights never depend on the
// preceding kernel, so they stream while that kernel drains and while this one quantizes its activations.
// Warps 0-7 consume: every warp takes block(s) `warp` of each slot straight from shared memory (a lane reads
// 128 bits = 4 columns x 8 k, a warp 512 contiguous bytes: conflict-free), feeds mma.sync.m16n8k32 (u8 x s8 ->
// s32, exact), scales per K group in fp32 and frees the slot with one mbarrier arrival per warp.
//
// Reduction.  At the end of a stripe the eight warps' partial sums meet in shared memory (double-buffered,
// one named barrier per stripe) and warp m adds row m in warp order: fixed order, no atomics, no global
// scratch.  With cs > 1 the CTA's sum goes over distributed shared memory into the inbox of the stripe's owner
// (rank = stripe mod cs), which adds the cs contributions in rank order after one cluster barrier.
//
// Activations.  Either quantized here (a warp takes 128 consecutive k of all rows; codes and scales bit-equal
// to FC_dynamic_quantize_x, ops/op_fc.hpp:246-268, group sums tree-ordered), or -- PREQ -- fetched, already
// quantized, with bulk copies (q4fc_quant_x_q8 / q4fc_rmsnorm_quant / q4fc_silu_mul_quant made them).
//
// Every wait is bounded (one second by %globaltimer): when it runs out the status word is set, the CTA's
// other waits end at once, all roles run to the end of their loops (no barrier is left waiting for anyone)
// and the kernel returns after a short pause for copies still in flight.
#pragma once
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"
#include "decode_math.cuh"

namespace cg = cooperative_groups;

namespace q4fc {
namespace {

constexpr int kRW = 8;  // consumer warps
constexpr int kRThreads = (kRW + 1) * 32;
constexpr int kRingMax = 10;  // most slots a ring can have
constexpr int kMaxJobs = 4;
constexpr int kMaxOwned = 16;  // stripes per cluster when cs > 1 (bounds the inbox)
constexpr unsigned long long kWaitLimitNs = 1000000000ull;

struct RingParams {
    const float* x;  // fp32 [rows][ldx]; TP with x_stamped: stamped 64-bit words [rows][ldx]
    int64_t K, ldx;
    int rows, rows_p;  // rows_p: rows rounded up to even
    int Kg, njobs;
    const uint8_t* wq[kMaxJobs];
    float* y[kMaxJobs];
    const float* addend[kMaxJobs];  // optional: y = fc(x) + addend; addend_ld = 0 broadcasts one row (a bias)
    int64_t N[kMaxJobs], ldy[kMaxJobs], addend_ld[kMaxJobs];
    int s_end[kMaxJobs];  // one past the last stripe of job i in the common stripe index space
    int cs, log2cs, nc;   // CTAs per cluster (power of two), clusters
    int sq, sr;           // stripes per cluster: sq, the first sr clusters one more
    int kq, kr;           // K groups per rank: kq, the first kr ranks one more
    int slice_k;          // elements of the widest K slice
    int code_stride;      // bytes between code rows in shared memory
    int depth, slot_bytes, ring_off;
    int inbox_stripes;  // stripes a CTA can own (cs > 1)
    int x_vec_ok;
    const int8_t* xq;  // PREQ: codes [rows][xq_stride], scales and group sums [Kg][16]
    const float* xsc;
    int64_t xq_stride;
    int* status;  // set non-zero when a bounded wait ran out
    // N-split over several GPUs (TP): outputs leave as 8-byte stamped words (fp32 value, low 32 bits of the step
    // counter) stored into every rank's buffer; a 64-bit store is indivisible, so a reader that finds the
    // current stamp has the value too
    int world, x_stamped;
    int64_t col_off[kMaxJobs];
    unsigned long long* y_peer[kMaxJobs][8];
    const unsigned long long* epoch;
};

// ---- PTX wrappers -------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> this CTA's shared memory; bytes % 16 == 0, both addresses 16-byte aligned
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void consumer_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kRW * 32) : "memory"); }

// Bounded wait on an mbarrier phase.  Once one wait of the CTA has run out (*fail != 0) all others end at once.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* fail, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return;
    const unsigned long long t0 = globaltimer_ns();
    for (unsigned it = 1;; it++) {
        if (mbar_try_wait(bar, parity)) return;
        if ((it & 255) == 0) {
            if (*fail != 0) return;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
                *fail = 1;
                atomicCAS(status, 0, code);
                return;
            }
        }
    }
}

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

// ---- the eight consumer warps quantize this CTA's K slice of the rows (ops/op_fc.hpp:246-268) ------------------
template <int G, int ROWS, bool SIGNED, bool TP>
__device__ __forceinline__ void quantize_slice(const RingParams& p, int warp, int lane, int k0, int Kc, uint8_t* codes,
                                               float* sc, uint32_t stamp) {
    constexpr int SEG = G / 4;    // lanes per group
    constexpr int GPC = 128 / G;  // groups per 128-k chunk
    const int Ls = Kc * G;        // slice length per row
    const int64_t kbase = (int64_t)k0 * G;
    const int chunks = (Ls + 127) >> 7;
    for (int ch = warp; ch < chunks; ch += kRW) {
        const int e = ch * 128 + lane * 4;  // element inside the slice
        const int64_t k = kbase + e;
        const int kbl = ch * GPC + lane / SEG;
        const bool exists = kbl < Kc;
        const int len = exists ? (int)min((int64_t)G, p.K - (kbase + (int64_t)kbl * G)) : 0;
        const bool vec = p.x_vec_ok && (e < Ls) && (k + 4 <= p.K);
        float v[ROWS][4];
        bool late = false;
#pragma unroll
        for (int m = 0; m < ROWS; m++) {
            v[m][0] = v[m][1] = v[m][2] = v[m][3] = 0.0f;
            if (TP && m < p.rows && e < Ls && p.x_stamped) {
                // first try; words whose stamp is not this step's are re-read below
                const unsigned long long* src = reinterpret_cast<const unsigned long long*>(p.x) + m * p.ldx + k;
#pragma unroll
                for (int jj = 0; jj < 4; jj++)
                    if (k + jj < p.K) {
                        const unsigned long long w = ld_stamped(src + jj);
                        v[m][jj] = __uint_as_float((uint32_t)w);
                        late |= (uint32_t)(w >> 32) != stamp;
                    }
            } else if (m < p.rows && e < Ls) {
                const float* src = p.x + m * p.ldx + k;
                if (vec) {
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(src));
                    v[m][0] = a.x, v[m][1] = a.y, v[m][2] = a.z, v[m][3] = a.w;
                } else {
#pragma unroll
                    for (int jj = 0; jj < 4; jj++)
                        if (k + jj < p.K) v[m][jj] = __ldcg(src + jj);
                }
            }
        }
        if (TP && p.x_stamped) {
            if (late) {
                // some producer has not delivered yet: poll this lane's words, within the time limit
                const unsigned long long t0 = globaltimer_ns();
                for (unsigned it = 1; late; it++) {
                    late = false;
                    for (int m = 0; m < ROWS; m++) {
                        if (m >= p.rows) break;
                        const unsigned long long* src = reinterpret_cast<const unsigned long long*>(p.x) + m * p.ldx + k;
                        for (int jj = 0; jj < 4; jj++)
                            if (k + jj < p.K) {
                                const unsigned long long w = ld_stamped(src + jj);
                                v[m][jj] = __uint_as_float((uint32_t)w);
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
        uint32_t packed[ROWS];
        float d[ROWS], aux[ROWS];
        q8_quantize_rows<G, ROWS, SIGNED>(v, lane, len, packed, d, aux);
        if (exists) {
#pragma unroll
            for (int m = 0; m < ROWS; m++)
                if (m < p.rows) {
                    *reinterpret_cast<uint32_t*>(codes + m * p.code_stride + e) = packed[m];
                    if (lane % SEG == 0) {
                        sc[kbl * 16 + m * 2 + 0] = d[m];
                        sc[kbl * 16 + m * 2 + 1] = aux[m];
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
    // [0,256): mbarriers full[kRingMax], empty[kRingMax], xbar; failure flag at 192
    // then part [2][kRW][rows_p*32] f32 | inbox [inbox_stripes][cs][rows_p*32] f32 (cs > 1) | sc [kc_max][16] f32
    //      | codes [rows][code_stride] | ring [depth][slot_bytes]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int cs = p.cs;
    const int j = (int)(blockIdx.x & (cs - 1));  // rank in the cluster (clusters are consecutive CTAs)
    const int c = (int)(blockIdx.x >> p.log2cs);
    const int s0 = c * p.sq + min(c, p.sr);
    const int r = p.sq + (c < p.sr ? 1 : 0);
    const int k0 = j * p.kq + min(j, p.kr);
    const int Kc = p.kq + (j < p.kr ? 1 : 0);  // >= 1: the launcher keeps cs <= Kg
    const int kc_max = p.slice_k / G;
    const int slot_f = p.rows_p * 32;

    const uint32_t bar0 = smem_u32(smem);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kRingMax + s); };
    const uint32_t xbar = bar0 + 8u * (2 * kRingMax);
    volatile int* fail = reinterpret_cast<volatile int*>(smem + 192);
    float* part = reinterpret_cast<float*>(smem + 256);
    float* inbox = part + 2 * kRW * slot_f;
    float* sc = inbox + (cs > 1 ? p.inbox_stripes * cs * slot_f : 0);
    uint8_t* codes = reinterpret_cast<uint8_t*>(sc + kc_max * 16);
    uint8_t* ring = smem + p.ring_off;
    const int depth = p.depth;

    cg::cluster_group cluster = cg::this_cluster();

    if (threadIdx.x == kRW * 32) {
        for (int i = 0; i < depth; i++) {
            mbar_init(full_bar(i), 1);
            mbar_init(empty_bar(i), kRW);
        }
        mbar_init(xbar, 1);
        *fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    pdl_launch_dependents();
    // "this CTA runs": nobody may store into a CTA's shared memory before that CTA has started
    if (cs > 1) cluster_arrive_release();

    // the stripe's job, its weights and its index inside that job
    auto job_of = [&](int sg, int& ls) {
        int jb = 0;
        while (jb + 1 < p.njobs && sg >= p.s_end[jb]) jb++;
        ls = sg - (jb ? p.s_end[jb - 1] : 0);
        return jb;
    };

    const int slots_per_stripe = (Kc + SB - 1) / SB;
    const int total_slots = r * slots_per_stripe;

    // ---- producer state (used by one thread)
    int p_li = 0, p_kb = 0, p_s = 0, p_issued = 0;
    auto issue_slot = [&]() {
        const int nblk = min(SB, Kc - p_kb);
        const uint32_t bytes = (uint32_t)nblk * BS;
        int ls;
        const int jb = job_of(s0 + p_li, ls);
        const uint8_t* src = p.wq[jb] + ((int64_t)ls * p.Kg + k0 + p_kb) * BS;
        mbar_expect_tx(full_bar(p_s), bytes);
        bulk_g2s(smem_u32(ring + (size_t)p_s * p.slot_bytes), src, bytes, full_bar(p_s));
        p_kb += SB;
        if (p_kb >= Kc) p_kb = 0, p_li++;
        if (++p_s == depth) p_s = 0;
        p_issued++;
    };

    uint32_t stamp = 0;
    if (warp == kRW) {
        if (lane == 0) {
            // weights do not depend on the preceding kernel: fill the ring now
            const int first = min(depth, total_slots);
            for (int i = 0; i < first; i++) issue_slot();
            if constexpr (PREQ) {
                pdl_wait_prior_grid();
                // this CTA's K slice of the quantized activations
                const uint32_t row_bytes = (uint32_t)(Kc * G);
                mbar_expect_tx(xbar, row_bytes * p.rows + (uint32_t)Kc * 64u);
                for (int m = 0; m < p.rows; m++)
                    bulk_g2s(smem_u32(codes + m * p.code_stride), p.xq + (int64_t)m * p.xq_stride + (int64_t)k0 * G,
                             row_bytes, xbar);
                bulk_g2s(smem_u32(sc), p.xsc + (int64_t)k0 * 16, (uint32_t)Kc * 64u, xbar);
            }
        }
    } else {
        pdl_wait_prior_grid();
        if constexpr (TP) stamp = (uint32_t)*reinterpret_cast<const volatile unsigned long long*>(p.epoch);
        if constexpr (!PREQ) quantize_slice<G, ROWS, SIGNED, TP>(p, warp, lane, k0, Kc, codes, sc, stamp);
    }
    __syncwarp();
    __syncthreads();  // barriers initialised; codes and scales of the slice written (fused quantizer)
    if (cs > 1) cluster_wait_acquire();  // every CTA of the cluster runs: pushes are allowed

    if (warp == kRW) {
        if (lane == 0) {
            // refill: slot n reuses ring position n % depth once its consumers have freed it
            uint32_t eph = 0;  // parity of the empty barrier's completion to wait for
            int wrapped = 0;
            while (p_issued < total_slots) {
                mbar_wait(empty_bar(p_s), eph, fail, p.status, 0x52454D50);  // 'REMP'
                issue_slot();
                if (++wrapped == depth) wrapped = 0, eph ^= 1;
            }
        }
    } else {
        if constexpr (PREQ) mbar_wait(xbar, 0, fail, p.status, 0x52584251);  // 'RXBQ'
        const uint8_t* my_codes = codes + g * p.code_stride + 8 * t;
        const bool row_live = g < p.rows;
        int cs_ = 0;       // consumer ring position
        uint32_t fph = 0;  // parity of the full barrier's completion to wait for
        for (int li = 0; li < r; li++) {
            float acc[4][2];
#pragma unroll
            for (int i = 0; i < 4; i++) acc[i][0] = acc[i][1] = 0.0f;
            for (int kb0 = 0; kb0 < Kc; kb0 += SB) {
                mbar_wait(full_bar(cs_), fph, fail, p.status, 0x5246554C);  // 'RFUL'
                const int nblk = min(SB, Kc - kb0);
                const uint8_t* slot = ring + (size_t)cs_ * p.slot_bytes;
#pragma unroll
                for (int i = 0; i < NBLK; i++) {
                    const int b = warp * NBLK + i;
                    if (b < nblk) {
                        const uint8_t* blk = slot + b * BS;
                        uint4 q[SETS];
#pragma unroll
                        for (int jj = 0; jj < SETS; jj++)
                            q[jj] = *reinterpret_cast<const uint4*>(blk + (4 * jj + t) * 128 + g * 16);
                        const uint2 wd = *reinterpret_cast<const uint2*>(blk + 16 * G + g * 8);
                        uint2 wm = make_uint2(0u, 0u);
                        if (QTYPE == 1) wm = *reinterpret_cast<const uint2*>(blk + 16 * G + 64 + g * 8);
                        const int ck = kb0 + b;
                        block_accumulate<G, QTYPE, SIGNED>(q, wd, wm, my_codes + ck * G, row_live, sc + ck * 16, t, acc);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(cs_));
                if (++cs_ == depth) cs_ = 0, fph ^= 1;
            }
            // ---- the stripe's slice is done: the warps' partial sums meet in shared memory
            float* pw = part + ((li & 1) * kRW + warp) * slot_f;
#pragma unroll
            for (int mi = 0; mi < 2; mi++)
                if ((2 * t + mi) < p.rows_p)
                    *reinterpret_cast<float4*>(pw + (2 * t + mi) * 32 + g * 4) =
                        make_float4(acc[0][mi], acc[1][mi], acc[2][mi], acc[3][mi]);
            consumer_bar_sync();
            // warp m adds row m in warp order.  The buffer of stripe li is written again at stripe li + 2, which
            // no thread reaches before every thread has passed the barrier of stripe li + 1, i.e. finished here.
            if (warp < p.rows) {
                const float* src = part + (li & 1) * kRW * slot_f + warp * 32 + lane;
                float sum = src[0];
#pragma unroll
                for (int w = 1; w < kRW; w++) sum += src[w * slot_f];
                if (cs > 1) {
                    float* dst = inbox + (((li >> p.log2cs) << p.log2cs) + j) * slot_f + warp * 32 + lane;
                    const int owner = li & (cs - 1);
                    if (owner != j) dst = cluster.map_shared_rank(dst, owner);
                    *dst = sum;
                } else {
                    int ls;
                    const int jb = job_of(s0 + li, ls);
                    const int64_t n = (int64_t)ls * 32 + lane;
                    if (n < p.N[jb]) {
                        if (p.addend[jb] != nullptr) sum = __fadd_rn(sum, p.addend[jb][warp * p.addend_ld[jb] + n]);
                        if constexpr (!TP) {
                            p.y[jb][warp * p.ldy[jb] + n] = sum;
                        } else {
                            for (int rk = 0; rk < p.world; rk++)
                                st_stamped(p.y_peer[jb][rk] + warp * p.ldy[jb] + p.col_off[jb] + n, sum, stamp);
                        }
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
        if (warp < p.rows) {  // consumer warp m: row m
            for (int li = j; li < r; li += cs) {
                const float* src = inbox + ((li >> p.log2cs) << p.log2cs) * slot_f + warp * 32 + lane;
                float sum = src[0];
                for (int q = 1; q < cs; q++) sum += src[q * slot_f];
                int ls;
                const int jb = job_of(s0 + li, ls);
                const int64_t n = (int64_t)ls * 32 + lane;
                if (n < p.N[jb]) {
                    if (p.addend[jb] != nullptr) sum = __fadd_rn(sum, p.addend[jb][warp * p.addend_ld[jb] + n]);
                    if constexpr (!TP) {
                        p.y[jb][warp * p.ldy[jb] + n] = sum;
                    } else {
                        for (int rk = 0; rk < p.world; rk++)
                            st_stamped(p.y_peer[jb][rk] + warp * p.ldy[jb] + p.col_off[jb] + n, sum, stamp);
                    }
                }
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

// The pre-quantized form has one instantiation per block type (nothing in it depends on the row count at
// compile time)
template <int G, int QTYPE, bool SIGNED, bool TP>
RingVariant* ring_variant_for_rows(int rows, bool preq) {
    if (preq) return ring_variant_of<G, QTYPE, SIGNED, 8, TP, true>();
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

// Above this many activation values (rows x K) a separate quantizing launch in front of the FC beats the
// quantizer inside it, which every CTA (or cluster) runs for itself.  Needs scratch: used only when the
// caller's workspace has room for it.  Measured on Llama-7B shapes: it pays when the per-CTA share of the
// quantization is the long pole -- K = 11008 at 4 and 8 rows.
constexpr int64_t kPreQuantMinValues = 40 * 1024;

// what the FC entry points hand to the launcher per weight tensor
struct RingJob {
    const uint8_t* wq;
    int64_t Ng, N;
    float* y;
    int64_t ldy;
    const float* addend;
    int64_t addend_ld;
};

template <bool TP>
int launch_ring_impl(const float* x, int rows, int64_t K, int64_t ldx, int64_t Kg, int qtype, int G,
                     const RingJob* jobs, int njobs, unsigned flags, cudaStream_t s, const q4fc_tp_site* const* tp,
                     void* ws, size_t ws_bytes, const void* xq_given) {
    if (rows == 0) return Q4FC_OK;
    const DeviceInfo* di = device_info();
    if (!di) return Q4FC_ECUDA;
    RingParams p = {};
    int64_t ng_total = 0;
    p.njobs = 0;
    for (int i = 0; i < njobs; i++) {
        // a tensor (or a rank's shard) without columns takes no part
        if (jobs[i].N == 0 || jobs[i].Ng == 0) continue;
        const int k = p.njobs++;
        p.wq[k] = jobs[i].wq, p.y[k] = jobs[i].y, p.addend[k] = jobs[i].addend;
        p.N[k] = jobs[i].N, p.ldy[k] = jobs[i].ldy, p.addend_ld[k] = jobs[i].addend_ld;
        ng_total += jobs[i].Ng;
        if (ng_total * Kg >= 0x7fffffffLL) {
            set_error("fc_decode: %lld blocks exceed the 2^31 limit", (long long)(ng_total * Kg));
            return Q4FC_ELIMIT;
        }
        p.s_end[k] = (int)ng_total;
        if (TP) {
            const q4fc_tp_site* t = tp[i];
            p.col_off[k] = t->col_off;
            for (int rk = 0; rk < t->world; rk++) p.y_peer[k][rk] = t->y_peer[rk];
        }
    }
    if (p.njobs == 0) return Q4FC_OK;
    for (int k = p.njobs; k < kMaxJobs; k++) p.s_end[k] = (int)ng_total;
    p.x = x, p.K = K, p.ldx = ldx, p.rows = rows, p.rows_p = (rows + 1) / 2 * 2, p.Kg = (int)Kg;
    int* status = ws ? static_cast<int*>(ws) : ring_status_word();
    if (TP) {
        p.world = tp[0]->world, p.x_stamped = tp[0]->x_stamped, p.epoch = tp[0]->epoch;
        status = tp[0]->status;
    }
    if (!status) return Q4FC_ECUDA;
    p.status = status;
    const bool sgn = (flags & Q4FC_FLAG_NIBBLE_SIGNED) && qtype == 0;
    const bool pdl = (flags & Q4FC_FLAG_PDL) != 0;

    // pre-quantized input: scratch at its fixed place in the workspace, behind what the stream-K form uses
    bool preq = false, own_quant_launch = false;
    p.xq_stride = Kg * G;
    const uint8_t* xq_base = nullptr;
    if (TP && tp[0]->xq_scratch != nullptr && !tp[0]->x_stamped) {
        // multi-GPU form with a plain input: quantize once into the caller's scratch, in front of the FC kernel
        xq_base = static_cast<const uint8_t*>(tp[0]->xq_scratch);
        preq = own_quant_launch = true;
    } else if (!TP && xq_given != nullptr) {
        // the caller quantized the activations already (q4fc_quant_x_q8 / q4fc_rmsnorm_quant / ...)
        xq_base = static_cast<const uint8_t*>(xq_given);
        preq = true;
    } else if (!TP && ws != nullptr && ((flags & Q4FC_FLAG_PREQUANT) || (int64_t)rows * K >= kPreQuantMinValues) &&
               ws_bytes >= decode_prequant_offset() + quant_pre_bytes(rows, K, G)) {
        xq_base = static_cast<uint8_t*>(ws) + decode_prequant_offset();
        preq = own_quant_launch = true;
    }
    if (preq) {
        p.xq = reinterpret_cast<const int8_t*>(xq_base);
        p.xsc = reinterpret_cast<const float*>(xq_base + align_up((size_t)(rows * Kg * G), 256));
    }
    RingVariant* v = ring_pick_variant<TP>(qtype, G, sgn, rows, preq);
    int dev = 0;
    Q4FC_CUDA_OK(cudaGetDevice(&dev));
    if (dev >= 64) {
        set_error("fc_decode: device index %d beyond the 64 this library keeps state for", dev);
        return Q4FC_ELIMIT;
    }

    // ---- shape of the launch: K split (clusters) only when the stripes alone cannot fill the GPU
    const int sms = di->sm_count;
    const int BS = block_bytes(qtype, G);
    const int SB = kRW * (G == 32 ? 4 : 1);
    p.slot_bytes = SB * BS;
    int cs = 1;
    while (cs < 8 && cs * 2 <= Kg && ng_total * cs * 2 <= sms) cs *= 2;
    size_t fixed = 0;
    int kc_max = 0, nc = 0;
    for (;; cs *= 2) {
        p.cs = cs;
        p.log2cs = 0;
        while ((1 << p.log2cs) < cs) p.log2cs++;
        p.kq = (int)(Kg / cs), p.kr = (int)(Kg % cs);
        kc_max = p.kq + (p.kr > 0 ? 1 : 0);
        p.slice_k = kc_max * G;
        p.code_stride = (p.slice_k + 127) / 128 * 128 + 32;  // rows 32 B apart modulo 128: conflict-free 8-byte operand loads
        int nc_cap = sms / cs;
        if (cs > 1) {
            std::lock_guard<std::mutex> lk(g_setup_mutex);
            if (v->max_clusters[dev][p.log2cs] == 0) {
                if (!v->attr_done[dev]) {
                    Q4FC_CUDA_OK(cudaFuncSetAttribute(v->fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      di->max_smem_optin));
                    v->attr_done[dev] = true;
                }
                cudaLaunchConfig_t cfg;
                cudaLaunchAttribute attr[2];
                // queried at the largest footprint a CTA can have: one CTA per SM either way
                ring_fill_launch_config(cfg, attr, cs, cs, (size_t)di->max_smem_optin, false, nullptr);
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, v->fn, &cfg) != cudaSuccess || n <= 0) {
                    cudaGetLastError();
                    n = sms / cs / 2;  // conservative stand-in
                    if (n < 1) n = 1;
                }
                v->max_clusters[dev][p.log2cs] = n;
            }
            nc_cap = v->max_clusters[dev][p.log2cs];
        }
        // all clusters resident at once (one wave); with cs > 1 at most kMaxOwned stripes per cluster
        nc = (int)(ng_total < nc_cap ? ng_total : nc_cap);
        if (cs > 1) {
            const int64_t nc_lo = (ng_total + kMaxOwned - 1) / kMaxOwned;
            if (nc < nc_lo) nc = (int)nc_lo;  // more than one wave: only for shapes no caller should split this way
        }
        p.nc = nc;
        p.sq = (int)(ng_total / nc), p.sr = (int)(ng_total % nc);
        const int r_max = p.sq + (p.sr > 0 ? 1 : 0);
        p.inbox_stripes = cs > 1 ? (r_max + cs - 1) / cs : 0;
        const size_t slot_f = (size_t)p.rows_p * 32;
        fixed = 256 + 2 * kRW * slot_f * 4 + (size_t)p.inbox_stripes * cs * slot_f * 4 + (size_t)kc_max * 64 +
                (size_t)rows * p.code_stride;
        fixed = align_up(fixed, 128);
        if (fixed + 2 * (size_t)p.slot_bytes <= (size_t)di->max_smem_optin) break;
        if (cs >= 8 || cs * 2 > Kg) {
            set_error("fc_decode: rows=%d K=%lld needs %zu bytes of shared memory (limit %d)", rows, (long long)K,
                      fixed + 2 * (size_t)p.slot_bytes, di->max_smem_optin);
            return Q4FC_ELIMIT;
        }
    }
    p.ring_off = (int)fixed;
    {
        // as deep as the shared memory allows, but no deeper than the busiest CTA has slots
        const int r_max = p.sq + (p.sr > 0 ? 1 : 0);
        const int64_t want = (int64_t)r_max * ((kc_max + SB - 1) / SB);
        int64_t depth = ((int64_t)di->max_smem_optin - (int64_t)fixed) / p.slot_bytes;
        if (depth > kRingMax) depth = kRingMax;
        if (depth > want) depth = want;
        if (depth < 1) depth = 1;
        p.depth = (int)depth;
    }
    const size_t smem = fixed + (size_t)p.depth * p.slot_bytes;
    p.x_vec_ok = (K % 4 == 0) && (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    {
        std::lock_guard<std::mutex> lk(g_setup_mutex);
        if (!v->attr_done[dev]) {
            Q4FC_CUDA_OK(cudaFuncSetAttribute(v->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin));
            v->attr_done[dev] = true;
        }
    }
    if (own_quant_launch) {
        if (int rc = launch_quant_x_pre(x, rows, K, ldx, G, sgn, const_cast<int8_t*>(p.xq), const_cast<float*>(p.xsc),
                                        pdl, s))
            return rc;
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    // behind its own quantizing launch the FC always starts early: its weight copies run beside that launch
    ring_fill_launch_config(cfg, attr, p.nc * p.cs, p.cs, smem, pdl || own_quant_launch, s);
    void* args[] = {const_cast<RingParams*>(&p)};
    Q4FC_CUDA_OK(cudaLaunchKernelExC(&cfg, v->fn, args));
    return Q4FC_OK;
}

}  // namespace
}  // namespace q4fc
