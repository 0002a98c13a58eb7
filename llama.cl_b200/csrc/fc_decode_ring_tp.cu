// Multi-GPU instantiations of the decode kernel (fc_decode_ring_impl.cuh, TP = true): outputs leave as
// epoch-stamped 64-bit words stored into every rank's buffer, inputs may be such a buffer.  Also the two
// small kernels around them: the step barrier and the unpacking of a stamped buffer.
#include "fc_decode_ring_impl.cuh"

namespace q4fc {
namespace {

struct StepArgs {
    unsigned long long* epoch;
    unsigned long long* barrier_peer[8];
    const unsigned long long* barrier_local;
    int world;
    int* status;
};

// Bounded spin until *counter >= target.  When the limit runs out the status word is set and the caller
// carries on with what is there; once the status word is set, later waits return at once, so that a lost
// rank costs one time limit and not one per kernel.
__device__ __forceinline__ void wait_for_arrivals(const unsigned long long* counter, unsigned long long target,
                                                  int* status, int code) {
    unsigned long long seen;
    const unsigned long long t0 = globaltimer_ns();
    for (unsigned it = 0;; it++) {
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(counter) : "memory");
        if (seen >= target) return;
        if ((it & 63) == 63) {
            if (*reinterpret_cast<volatile int*>(status) != 0) return;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
                atomicCAS(status, 0, code);
                return;
            }
        }
    }
}

// One warp.  Everything this rank launched before is complete (plain stream order), so announcing
// the new epoch to every rank and waiting for all of theirs separates the steps on all GPUs.
__global__ void tp_step_begin_kernel(const StepArgs a) {
    unsigned long long e = 0;
    if (threadIdx.x == 0) {
        e = *a.epoch + 1;
        *a.epoch = e;
    }
    __threadfence_system();
    __syncwarp();
    if ((int)threadIdx.x < a.world)
        asm volatile("red.release.sys.global.add.u64 [%0], 1;" ::"l"(a.barrier_peer[threadIdx.x]) : "memory");
    if (threadIdx.x == 0) wait_for_arrivals(a.barrier_local, e * (unsigned long long)a.world, a.status, 0x54504252);
}

// Unpacks a stamped buffer [rows, ld] into plain floats [rows, ldd], waiting (bounded) for every word to
// carry the current epoch: the hand-over to consumers that are not FC kernels.
__global__ void tp_collect_kernel(const unsigned long long* src, int rows, int64_t N, int64_t ld, float* dst,
                                  int64_t ldd, const unsigned long long* epoch, int* status) {
    const uint32_t stamp = (uint32_t)*reinterpret_cast<const volatile unsigned long long*>(epoch);
    const int64_t total = (int64_t)rows * N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / N, n = i - m * N;
        unsigned long long w = ld_stamped(src + m * ld + n);
        if ((uint32_t)(w >> 32) != stamp) {
            const unsigned long long t0 = globaltimer_ns();
            for (unsigned it = 1;; it++) {
                w = ld_stamped(src + m * ld + n);
                if ((uint32_t)(w >> 32) == stamp) break;
                if ((it & 63) == 0) {
                    if (*reinterpret_cast<volatile int*>(status) != 0) break;
                    if (globaltimer_ns() - t0 > kWaitLimitNs) {
                        atomicCAS(status, 0, 0x54505754);  // 'TPWT'
                        break;
                    }
                }
            }
        }
        dst[m * ldd + n] = __uint_as_float((uint32_t)w);
    }
}

struct CollectArgs {
    const unsigned long long* src[16];
    float* dst[16];
    int64_t N[16], ld[16], ldd[16];
    int64_t end[16];  // one past the last word of buffer i in the launch's common index space
    int n;
};

// tp_collect_kernel over several buffers; dst == nullptr: only wait for the buffer's words
__global__ void tp_collect_multi_kernel(const CollectArgs a, const unsigned long long* epoch, int* status) {
    const uint32_t stamp = (uint32_t)*reinterpret_cast<const volatile unsigned long long*>(epoch);
    const int64_t total = a.end[a.n - 1];
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int b = 0;
        while (i >= a.end[b]) b++;
        const int64_t r = i - (b ? a.end[b - 1] : 0);
        const int64_t m = r / a.N[b], n = r - m * a.N[b];
        const unsigned long long* p = a.src[b] + m * a.ld[b] + n;
        unsigned long long w = ld_stamped(p);
        if ((uint32_t)(w >> 32) != stamp) {
            const unsigned long long t0 = globaltimer_ns();
            for (unsigned it = 1;; it++) {
                w = ld_stamped(p);
                if ((uint32_t)(w >> 32) == stamp) break;
                if ((it & 63) == 0) {
                    if (*reinterpret_cast<volatile int*>(status) != 0) break;
                    if (globaltimer_ns() - t0 > kWaitLimitNs) {
                        atomicCAS(status, 0, 0x54505754);  // 'TPWT'
                        break;
                    }
                }
            }
        }
        if (a.dst[b] != nullptr) a.dst[b][m * a.ldd[b] + n] = __uint_as_float((uint32_t)w);
    }
}

}  // namespace

int launch_fc_decode_ring_tp_batch(const q4fc_tp_call* calls, const q4fc_tp_site* const* sites, int ncalls, int qtype,
                                   int G, unsigned flags, cudaStream_t s) {
    RingCall c[kMaxTpJobs];
    for (int i = 0; i < ncalls; i++)
        c[i] = {static_cast<const float*>(calls[i].x), calls[i].ldx, calls[i].xq, (int)calls[i].rows, calls[i].K,
                calls[i].Kg, static_cast<const uint8_t*>(calls[i].wq), calls[i].Ng, calls[i].N, nullptr, calls[i].ldy,
                nullptr, 0};
    return launch_ring_impl<true>(c, ncalls, qtype, G, flags, s, sites, nullptr, 0);
}

int launch_tp_collect_multi(const unsigned long long* const* src, const int64_t* rows, const int64_t* N,
                            const int64_t* ld, float* const* dst, const int64_t* ldd, int n,
                            const unsigned long long* epoch, int* status, cudaStream_t s) {
    CollectArgs a = {};
    int64_t total = 0;
    int k = 0;
    for (int i = 0; i < n; i++) {
        if (rows[i] == 0 || N[i] == 0) continue;
        a.src[k] = src[i], a.dst[k] = dst ? dst[i] : nullptr, a.N[k] = N[i], a.ld[k] = ld[i];
        a.ldd[k] = (dst && dst[i]) ? ldd[i] : 0;
        total += rows[i] * N[i];
        a.end[k] = total;
        k++;
    }
    if (k == 0) return Q4FC_OK;
    a.n = k;
    const int64_t blocks = (total + 255) / 256;
    tp_collect_multi_kernel<<<(unsigned)(blocks < 1184 ? blocks : 1184), 256, 0, s>>>(a, epoch, status);
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

int launch_fc_decode_ring_tp(const float* x, int rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng,
                             int64_t Kg, int qtype, int G, int64_t N, int64_t ldy, unsigned flags, cudaStream_t s,
                             const q4fc_tp_site* tp) {
    const RingCall c = {x, ldx, nullptr, rows, K, Kg, wq, Ng, N, nullptr, ldy, nullptr, 0};
    return launch_ring_impl<true>(&c, 1, qtype, G, flags, s, &tp, nullptr, 0);
}

int launch_tp_step_begin(unsigned long long* epoch, unsigned long long* const* barrier_peer,
                         const unsigned long long* barrier_local, int world, int* status, cudaStream_t s) {
    StepArgs a;
    a.epoch = epoch, a.barrier_local = barrier_local, a.world = world, a.status = status;
    for (int i = 0; i < 8; i++) a.barrier_peer[i] = i < world ? barrier_peer[i] : nullptr;
    tp_step_begin_kernel<<<1, 32, 0, s>>>(a);
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

int launch_tp_collect(const unsigned long long* src, int64_t rows, int64_t N, int64_t ld, float* dst, int64_t ldd,
                      const unsigned long long* epoch, int* status, cudaStream_t s) {
    if (rows == 0 || N == 0) return Q4FC_OK;
    const int64_t blocks = (rows * N + 255) / 256;
    tp_collect_kernel<<<(unsigned)(blocks < 1184 ? blocks : 1184), 256, 0, s>>>(src, (int)rows, N, ld, dst, ldd, epoch,
                                                                             status);
    Q4FC_CUDA_OK(cudaGetLastError());
    return Q4FC_OK;
}

}  // namespace q4fc
