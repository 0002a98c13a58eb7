// Multi-GPU instantiations of the decode kernel (fc_decode_ring_impl.cuh, TP = true): outputs leave as
// epoch-stamped 64-bit words stored into every rank's buffer, inputs may be such a buffer.  Also the two
// small kernels around them: the step barrier and the unpacking of a stamped buffer.
#define Q4FC_TL_NAME q4fc_dbg_set_tl_tp
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

}  // namespace

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
