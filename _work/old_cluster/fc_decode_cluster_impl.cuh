// Decode FC (rows <= 8), cluster form: the default kernel behind q4fc_fc_decode, and with TP = true the
// kernel behind q4fc_fc_decode_tp.  Included by fc_decode_cluster.cu (TP = false) and
// fc_decode_cluster_tp.cu (TP = true): two translation units, so that the multi-GPU code paths cost the
// single-GPU instantiations nothing and the two sets compile side by side.
// Same arithmetic as fc_decode.cu (reference: fc_Q4A, ops/op_fc.hpp:286-426);
// what differs is how the work is cut and how partial sums meet.
//
// Decomposition.  A thread-block cluster of `cs` CTAs owns a contiguous range
// of stripes (32 output columns each).  CTA rank j of the cluster owns the K
// slice kb in [j*Kg/cs, (j+1)*Kg/cs) of every one of those stripes.  So
//   * a CTA only ever needs the activations of its own K slice: it quantizes
//     rows x K/cs values instead of rows x K (the quantization is spread over
//     the cluster with no redundancy inside it);
//   * partial sums of one stripe are pushed over distributed shared memory
//     into the CTA that owns the stripe's output (rank = stripe mod cs) and
//     added there in rank order after one cluster barrier -- no global
//     scratch, no atomics, fixed summation order.
// Inside a CTA the (stripes x K-slice) rectangle is flattened and split into
// equal contiguous runs per warp; a run is a sequence of `Kc`-block pieces,
// each piece contiguous in memory (Kc*BS bytes).
//
// Streaming.  As in fc_decode.cu a lane loads 128 bits of nibbles (4 columns
// x 8 k) straight from global memory and feeds mma.sync.m16n8k32 (u8 x s8 ->
// s32); two steps per warp are in flight in registers and both are issued
// before the programmatic-dependent-launch wait, because weights never depend
// on the preceding kernel.
//
// The two steps that follow the register steps are also requested into L2 with
// cp.async.bulk.prefetch before the wait; more than that evicts lines of the
// kernels running beside this one before they are used.
//
// Activations.  A warp reads 128 consecutive k of a row of the CTA's slice
// (one 128-bit load per lane, a few in flight) and quantizes them in
// registers by the rules of FC_dynamic_quantize_x (ops/op_fc.hpp:246-268,
// ops/utils.hpp:200-220): codes and scales bit-equal to the reference's, group
// sums tree-ordered.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

// Phase timestamps for tuning builds (-DQ4FC_TIMELINE): lane 0 of every warp records %globaltimer
// at phase boundaries into a buffer set with q4fc_debug_set_timeline().  Compiled out otherwise.
#ifdef Q4FC_TIMELINE
static __device__ long long* g_timeline = nullptr;
__device__ __forceinline__ long long gtime() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define Q4FC_MARK(k)                                                                       \
    do {                                                                                   \
        if (g_timeline && (threadIdx.x & 31) == 0)                                         \
            g_timeline[((long long)blockIdx.x * kCW + (threadIdx.x >> 5)) * 16 + (k)] = gtime(); \
    } while (0)
extern "C" __attribute__((visibility("default"))) int Q4FC_TIMELINE_SETTER(long long* buf) {
    return (int)cudaMemcpyToSymbol(g_timeline, &buf, sizeof(buf));
}
#else
#define Q4FC_MARK(k) \
    do {             \
    } while (0)
#endif

namespace q4fc {
namespace {

constexpr int kCW = 4;  // warps per CTA
constexpr int kCThreads = kCW * 32;
constexpr int kMaxStripes = 16;  // stripes per cluster (bounds the shared-memory inbox)
constexpr int kPrefetchSteps = 2;  // steps beyond the two in registers that a warp requests into L2 at its start
constexpr uint32_t kNibMask = 0x0F0F0F0Fu;

struct ClusterParams {
    const float* x;
    float* y;
    const uint8_t* wq;
    int64_t K, ldx, N, ldy;
    int rows, Ng, Kg;
    int cs, log2cs, nc;  // CTAs per cluster (a power of two), clusters
    int sq, sr;          // stripes per cluster: sq, the first sr clusters one more
    int kq, kr;          // K groups per rank: kq, the first kr ranks one more
    int slice_k;         // elements of the widest K slice: (kq + (kr > 0)) * G
    int code_stride;     // bytes between code rows in shared memory
    int pmax;            // most warps that can share one stripe's slice inside a CTA
    int slot_f;          // floats per inbox slot: 32 columns x rows (rounded up to 2)
    int inbox_slots;     // per-CTA inbox: owned stripes x cs x pmax slots
    int x_vec_ok;
    // activations quantized beforehand by quant_x_pre_kernel (PREQ instantiations): codes [rows][xq_stride],
    // scales and group sums [Kg][16]
    const int8_t* xq;
    const float* xsc;
    int64_t xq_stride;
    // optional epilogue: y = fc(x) + addend (the reference's iadd of a bias or of the residual stream after the FC,
    // chatllama/main.py:166-167, 356, 372).  addend_ld = 0: one row broadcast over the rows (bias); else row stride.
    const float* addend;
    int64_t addend_ld;
    // ---- N-split over several GPUs, joined by this kernel itself (world == 0: single GPU, fields unused).
    // Outputs travel as 8-byte "stamped" words: the fp32 value in the low half, the low 32 bits of the step
    // counter ("epoch") in the high half.  A 64-bit store is indivisible, so a reader that finds the current
    // epoch in the high half has the value too: no fence, no counter, no second message.  The owner of a
    // stripe stores its stamped outputs into the buffer of EVERY rank (peer-mapped pointers, plain stores
    // over NVLink) at column offset col_off.  A kernel whose input is such a buffer (x_stamped) re-reads each
    // word until the stamp is the current epoch.
    int world;
    int x_stamped;
    int64_t col_off;
    unsigned long long* y_peer[8];
    const unsigned long long* epoch;  // device scalar, advanced once per step by the step barrier
    int* status;                      // set to non-zero when a bounded wait ran out
};

constexpr unsigned long long kPeerWaitLimitNs = 1000000000ull;  // a wait on peers gives up after one second

// Bounded spin until *counter >= target.  When the limit runs out the status word is set and the caller
// carries on with what is there; once the status word is set, later waits return at once, so that a lost
// rank costs one time limit and not one per kernel.
__device__ __forceinline__ void wait_for_arrivals(const unsigned long long* counter, unsigned long long target,
                                                  int* status, int code) {
    unsigned long long seen, t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (unsigned it = 0;; it++) {
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(counter) : "memory");
        if (seen >= target) return;
        if ((it & 63) == 63) {
            if (*reinterpret_cast<volatile int*>(status) != 0) return;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > kPeerWaitLimitNs) {
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

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm(  // a pure function of its operands: left to the scheduler to interleave
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// request `bytes` (multiple of 16, 16-byte aligned) starting at p into L2; nothing waits for it
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// cluster barrier, split so that the arrival can be posted early
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

template <int G, int QTYPE>
struct Cl {
    static constexpr int BS = block_bytes(QTYPE, G);
    static constexpr int SETS = G / 32;
    static constexpr int NBLK = (G == 32) ? 4 : 1;
    struct Step {
        uint4 q[NBLK][SETS];
        uint2 wd[NBLK];
        uint2 wm[NBLK];
    };
};

template <int G, int QTYPE, bool SIGNED, int ROWS, bool TP, bool PREQ>
__global__ void __launch_bounds__(kCThreads, 4) fc_decode_cluster_kernel(const ClusterParams p) {
    using C = Cl<G, QTYPE>;
    constexpr int BS = C::BS;
    constexpr int SETS = C::SETS;
    constexpr int NBLK = C::NBLK;

    extern __shared__ __align__(16) uint8_t smem[];
    // [inbox: inbox_slots x slot_f f32][sc: kc_max x 16 f32][codes: rows x code_stride]
    float* inbox = reinterpret_cast<float*>(smem);
    float* sc = inbox + p.inbox_slots * p.slot_f;
    const int kc_max = p.slice_k / G;
    uint8_t* codes = reinterpret_cast<uint8_t*>(sc + kc_max * 16);

    cg::cluster_group cluster = cg::this_cluster();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int cs = p.cs;
    const int j = (int)(blockIdx.x & (cs - 1));  // rank in the cluster (clusters are consecutive CTAs)
    const int c = (int)(blockIdx.x >> p.log2cs);
    const int s0 = c * p.sq + min(c, p.sr);
    const int r = p.sq + (c < p.sr ? 1 : 0);
    const int k0 = j * p.kq + min(j, p.kr);
    const int Kc = p.kq + (j < p.kr ? 1 : 0);  // >= 1: the launcher keeps cs <= Kg
    const int F = r * Kc;
    const int f0 = (warp * F) / kCW;
    const int f1 = ((warp + 1) * F) / kCW;

    Q4FC_MARK(0);
    pdl_launch_dependents();

    // the inbox starts at zero (slots nobody writes to add nothing); first phase of the cluster
    // barrier: "my inbox is clean", posted before any load so that its release waits for nothing
    for (int i = threadIdx.x; i < p.inbox_slots * (p.slot_f / 4); i += kCThreads)
        reinterpret_cast<float4*>(inbox)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    Q4FC_MARK(8);
    if (cs > 1) cluster_arrive_release();
    Q4FC_MARK(9);

    // ---- weights: two steps in flight in registers, the rest of the run requested into L2
    typename C::Step cur, nxt;
    int fl = f0;                     // next block to load
    int li = f0 / Kc, lk = f0 - li * Kc;  // its (stripe, kb) inside the rectangle
    const int ci0 = li, ck0 = lk;
    const uint8_t* lane_base = p.wq + t * 128 + g * 16;
    auto load_step = [&](typename C::Step& s) {
#pragma unroll
        for (int i = 0; i < NBLK; i++) {
            if (fl < f1) {
                const uint8_t* blk = lane_base + ((int64_t)(s0 + li) * p.Kg + k0 + lk) * BS;
#pragma unroll
                for (int jj = 0; jj < SETS; jj++) s.q[i][jj] = ldg_stream_v4(blk + jj * 512);
                const uint8_t* tail = blk - t * 128 - g * 8 + 16 * G;  // wd of columns 4g..4g+3
                s.wd[i] = ldg_stream_v2(tail);
                if (QTYPE == 1) s.wm[i] = ldg_stream_v2(tail + 64);
                fl++;
                if (++lk == Kc) lk = 0, li++;
            }
        }
    };
    load_step(cur);
    load_step(nxt);
    Q4FC_MARK(10);
    // the next steps of the run are requested into L2 behind the register steps.  Measured: requesting the
    // whole run (the first form) costs 6 % on the sweep and on the token pass -- kernels that run side by side
    // then evict one another's lines before they are used; a window that rolls along with the loop is no
    // better than none; issuing the requests ahead of the register steps delays those by 7 %.
    const int f1p = min(f1, f0 + (2 + kPrefetchSteps) * NBLK);
    if (f1p - f0 > 2 * NBLK) {
        const int pf = f0 + 2 * NBLK;
        const int i_first = pf / Kc, i_last = (f1p - 1) / Kc;
        for (int i = i_first + lane; i <= i_last; i += 32) {  // one contiguous piece per stripe
            const int fb = max(pf, i * Kc), fe = min(f1p, (i + 1) * Kc);
            const uint8_t* a = p.wq + ((int64_t)(s0 + i) * p.Kg + k0 + (fb - i * Kc)) * BS;
            for (int done = 0; done < fe - fb; done += 16)
                l2_prefetch(a + (int64_t)done * BS, (uint32_t)(min(16, fe - fb - done) * BS));
        }
    }

    Q4FC_MARK(1);
    pdl_wait_prior_grid();
    uint32_t stamp = 0;
    if constexpr (TP) stamp = (uint32_t)*reinterpret_cast<const volatile unsigned long long*>(p.epoch);
    Q4FC_MARK(2);

    if constexpr (PREQ) {
        // ---- the activations were quantized by the launch before: fetch this CTA's K slice
        const int vec_per_row = Kc * (G / 16);
        const int8_t* src = p.xq + (int64_t)k0 * G;
        for (int i = threadIdx.x; i < p.rows * vec_per_row; i += kCThreads) {
            const int m = i / vec_per_row, c = i - m * vec_per_row;
            *reinterpret_cast<uint4*>(codes + m * p.code_stride + c * 16) =
                __ldcg(reinterpret_cast<const uint4*>(src + m * p.xq_stride) + c);
        }
        const float4* ssrc = reinterpret_cast<const float4*>(p.xsc) + (int64_t)k0 * 4;
        for (int i = threadIdx.x; i < Kc * 4; i += kCThreads) reinterpret_cast<float4*>(sc)[i] = __ldcg(ssrc + i);
    } else {
        // ---- quantize this CTA's K slice of the activation rows (ops/op_fc.hpp:246-268)
        constexpr int SEG = G / 4;    // lanes per group
        constexpr int GPC = 128 / G;  // groups per 128-k chunk
        const int Ls = Kc * G;        // slice length per row
        const int64_t kbase = (int64_t)k0 * G;
        const int chunks = (Ls + 127) >> 7;
        const int e0 = (lane % SEG) * 4;
        for (int ch = warp; ch < chunks; ch += kCW) {
            const int e = ch * 128 + lane * 4;  // element inside the slice
            const int64_t k = kbase + e;
            const int kbl = ch * GPC + lane / SEG;
            const bool exists = kbl < Kc;
            const int len = exists ? (int)min((int64_t)G, p.K - (kbase + (int64_t)kbl * G)) : 0;
            const int body = len & ~7;
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
                    unsigned long long t0, t1;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
                    for (unsigned it = 1; late; it++) {
                        late = false;
                        for (int m = 0; m < ROWS; m++) {
                            if (m >= p.rows) break;
                            const unsigned long long* src =
                                reinterpret_cast<const unsigned long long*>(p.x) + m * p.ldx + k;
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
                            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                            if (t1 - t0 > kPeerWaitLimitNs) {
                                atomicCAS(p.status, 0, 0x54505754);  // 'TPWT': carry on with what is there
                                break;
                            }
                        }
                    }
                }
                __syncwarp();
            }
            // all ROWS rows go through the same straight-line code (rows beyond p.rows are zero),
            // so the independent shuffle / divide chains of the rows overlap
            float amax[ROWS], fsum[ROWS];
#pragma unroll
            for (int m = 0; m < ROWS; m++) {
                amax[m] = 0.0f, fsum[m] = 0.0f;
#pragma unroll
                for (int jj = 0; jj < 4; jj++)
                    if (e0 + jj < len) {
                        amax[m] = fmaxf(amax[m], fabsf(v[m][jj]));
                        fsum[m] += v[m][jj];
                    }
            }
#pragma unroll
            for (int off = SEG / 2; off > 0; off >>= 1) {
#pragma unroll
                for (int m = 0; m < ROWS; m++) {
                    amax[m] = fmaxf(amax[m], __shfl_xor_sync(0xffffffffu, amax[m], off));
                    fsum[m] += __shfl_xor_sync(0xffffffffu, fsum[m], off);
                }
            }
#pragma unroll
            for (int m = 0; m < ROWS; m++) {
                const float d = div_const_rn(amax[m], 127.0f, 1.0f / 127.0f);
                const float id = inv_or_zero(d);
                uint32_t packed = 0;
                int isum = 0;
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    int q = 0;
                    if (e0 + jj < len) {
                        const float tq = __fmul_rn(v[m][jj], id);
                        if (e0 + jj < body) {
                            q = __float2int_rn(tq);  // 8-wide body of the reference: nearest even
                        } else {
                            const float h = __int_as_float((__float_as_int(tq) & 0x80000000) | 0x3F000000);
                            q = __float2int_rz(__fadd_rz(tq, h));  // its scalar tail: half away
                        }
                        q = min(127, max(-128, q));
                    }
                    isum += q;
                    packed |= (uint32_t)(q & 0xFF) << (8 * jj);
                }
                if (SIGNED) {
#pragma unroll
                    for (int off = SEG / 2; off > 0; off >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, off);
                }
                if (exists && m < p.rows) {
                    *reinterpret_cast<uint32_t*>(codes + m * p.code_stride + e) = packed;
                    if (e0 == 0) {
                        // the reference's 1/16 activation scale and x16 nibble shift of Q4_0 cancel exactly
                        sc[kbl * 16 + m * 2 + 0] = d;
                        sc[kbl * 16 + m * 2 + 1] = SIGNED ? __int_as_float(8 * isum) : fsum[m];
                    }
                }
            }
        }
    }
    Q4FC_MARK(3);
    __syncthreads();                     // codes and scales of the slice are ready (and this CTA's inbox is clean)
    if (cs > 1) cluster_wait_acquire();  // every inbox of the cluster is clean: pushes are allowed
    Q4FC_MARK(4);

    // ---- stream this warp's run; every finished piece is pushed to the stripe's owner:
    //      CTA (i mod cs), slot ((i / cs) * cs + sender rank) * warps + sender warp
    float acc[4][2];
#pragma unroll
    for (int i = 0; i < 4; i++) acc[i][0] = acc[i][1] = 0.0f;
    int f = f0;
    int ci = ci0, ck = ck0;  // compute cursor
    const uint8_t* my_codes = codes + g * p.code_stride + 8 * t;
    const bool row_live = g < p.rows;

    auto push = [&](int stripe_l) {
        // piece number = this warp's position among the warps that share the stripe's slice
        const int w_first = min(kCW - 1, (kCW * (stripe_l * Kc + 1) + F - 1) / F - 1);
        const int slot = (((stripe_l >> p.log2cs) << p.log2cs) + j) * p.pmax + (warp - w_first);
        float* dst = inbox + slot * p.slot_f;
        const int owner = stripe_l & (cs - 1);
        if (owner != j) dst = cluster.map_shared_rank(dst, owner);
#pragma unroll
        for (int mi = 0; mi < 2; mi++)
            if ((2 * t + mi) * 32 < p.slot_f)
                *reinterpret_cast<float4*>(dst + (2 * t + mi) * 32 + g * 4) =
                    make_float4(acc[0][mi], acc[1][mi], acc[2][mi], acc[3][mi]);
#pragma unroll
        for (int i = 0; i < 4; i++) acc[i][0] = acc[i][1] = 0.0f;
    };

    auto process = [&](const typename C::Step& st) {
#pragma unroll
        for (int i = 0; i < NBLK; i++) {
            if (f + i < f1) {
                // two accumulator chains per tile (even / odd row sets) halve the dependent-MMA latency
                int ia[4] = {0, 0, 0, 0}, ib[4] = {0, 0, 0, 0}, ja[4] = {0, 0, 0, 0}, jb[4] = {0, 0, 0, 0};
#pragma unroll
                for (int jj = 0; jj < SETS; jj++) {
                    uint2 xb = make_uint2(0u, 0u);
                    if (row_live) xb = *reinterpret_cast<const uint2*>(my_codes + ck * G + 32 * jj);
                    const uint4 q = st.q[i][jj];
                    uint32_t l0 = q.x & kNibMask, l1 = q.y & kNibMask, l2 = q.z & kNibMask, l3 = q.w & kNibMask;
                    uint32_t h0 = (q.x >> 4) & kNibMask, h1 = (q.y >> 4) & kNibMask, h2 = (q.z >> 4) & kNibMask,
                             h3 = (q.w >> 4) & kNibMask;
                    if (SIGNED) {
                        l0 ^= 0x08080808u, l1 ^= 0x08080808u, l2 ^= 0x08080808u, l3 ^= 0x08080808u;
                        h0 ^= 0x08080808u, h1 ^= 0x08080808u, h2 ^= 0x08080808u, h3 ^= 0x08080808u;
                    }
                    if (jj & 1) {
                        mma_u8s8(ja, l0, l1, h0, h1, xb.x, xb.y);
                        mma_u8s8(jb, l2, l3, h2, h3, xb.x, xb.y);
                    } else {
                        mma_u8s8(ia, l0, l1, h0, h1, xb.x, xb.y);
                        mma_u8s8(ib, l2, l3, h2, h3, xb.x, xb.y);
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; q++) ia[q] += ja[q], ib[q] += jb[q];
                const float4 s4 = *reinterpret_cast<const float4*>(sc + ck * 16 + t * 4);  // xs0, gs0, xs1, gs1
                const float2 wd01 = __half22float2(*reinterpret_cast<const __half2*>(&st.wd[i].x));
                const float2 wd23 = __half22float2(*reinterpret_cast<const __half2*>(&st.wd[i].y));
                const float wdf[4] = {wd01.x, wd01.y, wd23.x, wd23.y};
                const int iv[4][2] = {{ia[0], ia[1]}, {ia[2], ia[3]}, {ib[0], ib[1]}, {ib[2], ib[3]}};
                const float xs[2] = {s4.x, s4.z};
                const float gs[2] = {s4.y, s4.w};
                float wmf[4] = {0.f, 0.f, 0.f, 0.f};
                if (QTYPE == 1) {
                    const float2 wm01 = __half22float2(*reinterpret_cast<const __half2*>(&st.wm[i].x));
                    const float2 wm23 = __half22float2(*reinterpret_cast<const __half2*>(&st.wm[i].y));
                    wmf[0] = wm01.x, wmf[1] = wm01.y, wmf[2] = wm23.x, wmf[3] = wm23.y;
                }
#pragma unroll
                for (int cc = 0; cc < 4; cc++) {
#pragma unroll
                    for (int mi = 0; mi < 2; mi++) {
                        int I = iv[cc][mi];
                        if (SIGNED) I -= __float_as_int(gs[mi]);
                        acc[cc][mi] = fmaf(__fmul_rn(wdf[cc], xs[mi]), (float)I, acc[cc][mi]);
                        if (QTYPE == 1) acc[cc][mi] = fmaf(wmf[cc], gs[mi], acc[cc][mi]);
                    }
                }
                if (++ck == Kc) {  // end of this stripe's slice
                    push(ci);
                    ck = 0, ci++;
                }
            }
        }
    };

    while (true) {
        if (f >= f1) break;
        process(cur);
        f += NBLK;
        load_step(cur);
        if (f >= f1) break;
        process(nxt);
        f += NBLK;
        load_step(nxt);
    }
    if (ck != 0 && f1 > f0) push(ci);  // the run ended inside a stripe's slice
    Q4FC_MARK(5);

    // ---- every piece has been pushed: the owner adds its stripes in (rank, warp) order
    if (cs > 1) {
        cluster_arrive_release();
        cluster_wait_acquire();
    } else {
        __syncthreads();
    }
    Q4FC_MARK(6);
    for (int i = j + cs * warp; i < r; i += cs * kCW) {
        const float* src = inbox + ((i >> p.log2cs) << p.log2cs) * p.pmax * p.slot_f;
        const int64_t n = (int64_t)(s0 + i) * 32 + lane;
        const int nsl = cs * p.pmax;
#pragma unroll
        for (int m = 0; m < ROWS; m++) {
            if (m < p.rows) {
                float sum = 0.0f;
                for (int q = 0; q < nsl; q++) sum += src[q * p.slot_f + m * 32 + lane];
                if (n < p.N && p.addend != nullptr) sum = __fadd_rn(sum, p.addend[m * p.addend_ld + n]);
                if (n < p.N) {
                    if constexpr (!TP) {
                        p.y[m * p.ldy + n] = sum;
                    } else {
                        for (int rk = 0; rk < p.world; rk++)
                            st_stamped(p.y_peer[rk] + m * p.ldy + p.col_off + n, sum, stamp);
                    }
                }
            }
        }
    }
    Q4FC_MARK(7);
    // no CTA touches another CTA's shared memory after the barrier above, so exiting is safe
}

// one launchable instantiation: its function pointer plus lazily set attributes
struct Variant {
    const void* fn;
    bool attr_done[64];
    int max_clusters[64][4];  // [device][log2 cs], 0 = not queried yet
};

template <int G, int QTYPE, bool SIGNED, int ROWS, bool TP, bool PREQ>
Variant* variant_of() {
    static Variant v = {
        reinterpret_cast<const void*>(&fc_decode_cluster_kernel<G, QTYPE, SIGNED, ROWS, TP, PREQ>), {}, {}};
    return &v;
}

// The pre-quantized form has one instantiation per block type (its row loops run to 8 with a run-time bound)
template <int G, int QTYPE, bool SIGNED, bool TP>
Variant* variant_for_rows(int rows, bool preq) {
    if (preq) return variant_of<G, QTYPE, SIGNED, 8, TP, true>();
    if (rows <= 1) return variant_of<G, QTYPE, SIGNED, 1, TP, false>();
    if (rows <= 2) return variant_of<G, QTYPE, SIGNED, 2, TP, false>();
    if (rows <= 4) return variant_of<G, QTYPE, SIGNED, 4, TP, false>();
    return variant_of<G, QTYPE, SIGNED, 8, TP, false>();
}

template <bool TP>
Variant* pick_variant(int qtype, int G, bool sgn, int rows, bool preq) {
    if (qtype == 1 && G == 32) return variant_for_rows<32, 1, false, TP>(rows, preq);
    if (qtype == 1 && G == 128) return variant_for_rows<128, 1, false, TP>(rows, preq);
    if (qtype == 0 && G == 32 && !sgn) return variant_for_rows<32, 0, false, TP>(rows, preq);
    if (qtype == 0 && G == 128 && !sgn) return variant_for_rows<128, 0, false, TP>(rows, preq);
    if (qtype == 0 && G == 32) return variant_for_rows<32, 0, true, TP>(rows, preq);
    return variant_for_rows<128, 0, true, TP>(rows, preq);
}

void fill_launch_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int grid, int cs, size_t smem, bool pdl,
                        cudaStream_t s) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kCThreads);
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

// clusters of `cs` CTAs that can be resident at once (hardware placement included), cached
int max_resident_clusters(Variant* v, int dev, int cs, int log2cs, const DeviceInfo* di) {
    if (dev >= 64) return di->sm_count * 4 / cs;
    if (!v->attr_done[dev]) {
        if (cudaFuncSetAttribute(v->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin) !=
            cudaSuccess) {
            cudaGetLastError();
            return -1;
        }
        v->attr_done[dev] = true;
    }
    if (v->max_clusters[dev][log2cs] == 0) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[2];
        fill_launch_config(cfg, attr, cs, cs, 56 * 1024, false, nullptr);  // shared memory never exceeds this per CTA
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, v->fn, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = di->sm_count * 2 / cs;  // conservative stand-in
            if (n < 1) n = 1;
        }
        v->max_clusters[dev][log2cs] = n;
    }
    return v->max_clusters[dev][log2cs];
}


// Above this many activation values (rows x K) a separate quantizing launch in front of the FC beats the
// quantizer inside it, which every cluster runs for itself.  Needs scratch: used only when the caller's
// workspace has room for it.
// (pre_quant_min_values() returns kPreQuantMinValues unless the tuning variable Q4FC_PREQUANT_MIN_VALUES is set.)
// Measured on Llama-7B shapes: it pays when the per-CTA share of the quantization (rows x K / 8) is the long
// pole -- K = 11008 at 4 and 8 rows (15 -> 13 us, 21 -> 14 us per call) -- and not at K = 4096, where for wide
// outputs the extra launch competes with the weight stream the FC kernel has already requested.
constexpr int64_t kPreQuantMinValues = 40 * 1024;

template <bool TP>
int launch_cluster_impl(const float* x, int rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng, int64_t Kg,
                        int qtype, int G, int64_t N, float* y, int64_t ldy, unsigned flags, cudaStream_t s,
                        const q4fc_tp_site* tp, void* ws = nullptr, size_t ws_bytes = 0,
                        const void* xq_given = nullptr, const float* addend = nullptr, int64_t addend_ld = 0) {
    // a rank without columns still launches nothing: its peers count only the stripes that exist
    if (rows == 0 || N == 0) return Q4FC_OK;
    const DeviceInfo* di = device_info();
    if (!di) return Q4FC_ECUDA;
    if (Ng * Kg >= 0x7fffffffLL) {
        set_error("fc_decode: %lld blocks exceed the 2^31 limit", (long long)(Ng * Kg));
        return Q4FC_ELIMIT;
    }
    ClusterParams p;
    p.x = x, p.y = y, p.wq = wq;
    p.K = K, p.ldx = ldx, p.N = N, p.ldy = ldy;
    p.rows = rows, p.Ng = (int)Ng, p.Kg = (int)Kg;
    p.addend = addend, p.addend_ld = addend_ld;
    p.world = 0, p.x_stamped = 0, p.col_off = 0, p.epoch = nullptr, p.status = nullptr;
    for (int i = 0; i < 8; i++) p.y_peer[i] = nullptr;
    if (tp) {
        p.world = tp->world, p.x_stamped = tp->x_stamped, p.col_off = tp->col_off;
        for (int i = 0; i < tp->world; i++) p.y_peer[i] = tp->y_peer[i];
        p.epoch = tp->epoch, p.status = tp->status;
    }
    const bool sgn = (flags & Q4FC_FLAG_NIBBLE_SIGNED) && qtype == 0;
    const bool pdl = (flags & Q4FC_FLAG_PDL) != 0;
    // pre-quantized input: scratch at its fixed place in the workspace, behind what the stream-K form uses
    bool preq = false;
    p.xq = nullptr, p.xsc = nullptr, p.xq_stride = Kg * G;
    if (TP && tp->xq_scratch != nullptr && !tp->x_stamped) {
        // multi-GPU form with a plain input: quantize once into the caller's scratch, in front of the FC kernel
        uint8_t* base = static_cast<uint8_t*>(tp->xq_scratch);
        p.xq = reinterpret_cast<const int8_t*>(base);
        p.xsc = reinterpret_cast<const float*>(base + align_up((size_t)(rows * Kg * G), 256));
        preq = true;
    } else if (!TP && xq_given != nullptr) {
        // the caller quantized the activations already (q4fc_quant_x_q8 / q4fc_rmsnorm_quant)
        const uint8_t* base = static_cast<const uint8_t*>(xq_given);
        p.xq = reinterpret_cast<const int8_t*>(base);
        p.xsc = reinterpret_cast<const float*>(base + align_up((size_t)(rows * Kg * G), 256));
        preq = true;
    } else if (!TP && ws != nullptr && ((flags & Q4FC_FLAG_PREQUANT) || (int64_t)rows * K >= pre_quant_min_values()) &&
        (size_t)Ng * 4 <= kWsCounterCapacity && ws_bytes >= decode_prequant_offset() + quant_pre_bytes(rows, K, G)) {
        uint8_t* base = static_cast<uint8_t*>(ws) + decode_prequant_offset();
        p.xq = reinterpret_cast<const int8_t*>(base);
        p.xsc = reinterpret_cast<const float*>(base + align_up((size_t)(rows * Kg * G), 256));
        preq = true;
    }
    Variant* v = pick_variant<TP>(qtype, G, sgn, rows, preq);
    int dev = 0;
    Q4FC_CUDA_OK(cudaGetDevice(&dev));
    p.cs = 8;
    // Clusters of 8 spread the in-kernel quantization over more CTAs and give the shortest single call; when
    // the caller asks for the separate quantizing launch because calls run side by side, that reason is gone and
    // clusters of 4 (cheaper barriers, finer placement) are 4 % faster on the whole (and 13 % slower alone).
    if (preq && xq_given == nullptr && (TP || (flags & Q4FC_FLAG_PREQUANT))) p.cs = 4;
    while (p.cs > 1 && p.cs > Kg) p.cs /= 2;
    p.log2cs = 0;
    while ((1 << p.log2cs) < p.cs) p.log2cs++;
    int cap = max_resident_clusters(v, dev, p.cs, p.log2cs, di);
    if (cap < 0) return cuda_fail(cudaErrorUnknown, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
    // in a chain launched with programmatic serialization two kernels share the GPU: the next one
    // streams its weights toward L2 while this one finishes, so each takes half of the CTA slots (the whole or
    // three quarters of them measured 16 % / 12 % slower on a 225-call chain)
    if (pdl && cap >= 2) cap /= 2;
    p.nc = choose_cluster_count(Ng, cap);
    p.sq = (int)(Ng / p.nc), p.sr = (int)(Ng % p.nc);
    p.kq = (int)(Kg / p.cs), p.kr = (int)(Kg % p.cs);
    const int kc_max = p.kq + (p.kr > 0 ? 1 : 0);
    p.slice_k = kc_max * G;
    p.code_stride = (p.slice_k + 127) / 128 * 128 + 32;  // rows 32 B apart modulo 128: conflict-free 8-byte operand loads
    const int r_max = p.sq + (p.sr > 0 ? 1 : 0);
    p.pmax = (kCW + p.sq - 1) / p.sq + 1;  // a slice of Kc blocks meets at most ceil(kCW / r) + 1 warp runs
    if (p.pmax > kCW) p.pmax = kCW;
    p.slot_f = 32 * ((rows + 1) / 2 * 2);
    p.inbox_slots = (r_max + p.cs - 1) / p.cs * p.cs * p.pmax;  // owned stripes x senders x pieces
    p.x_vec_ok = (K % 4 == 0) && (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const size_t smem = (size_t)p.inbox_slots * p.slot_f * 4 + (size_t)kc_max * 64 + (size_t)rows * p.code_stride;
    if (smem > (size_t)di->max_smem_optin) {
        set_error("fc_decode: rows=%d K=%lld needs %zu bytes of shared memory (limit %d)", rows, (long long)K, smem,
                  di->max_smem_optin);
        return Q4FC_ELIMIT;
    }
    if (preq && xq_given == nullptr) {
        if (int rc = launch_quant_x_pre(x, rows, K, ldx, G, sgn, const_cast<int8_t*>(p.xq),
                                        const_cast<float*>(p.xsc), pdl, s))
            return rc;
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    // behind its own quantizing launch the FC always starts early: its weight loads run beside that launch
    fill_launch_config(cfg, attr, p.nc * p.cs, p.cs, smem, pdl || (preq && xq_given == nullptr), s);
    void* args[] = {const_cast<ClusterParams*>(&p)};
    Q4FC_CUDA_OK(cudaLaunchKernelExC(&cfg, v->fn, args));
    return Q4FC_OK;
}

}  // namespace
}  // namespace q4fc
