// Single-GPU instantiations of the decode kernel (fc_decode_ring_impl.cuh, TP = false), and the status
// word its kernels use when the caller passes no workspace.
#include "fc_decode_ring_impl.cuh"

namespace q4fc {

namespace {
// set non-zero by a kernel whose bounded wait ran out and that was launched without a workspace
__device__ int g_ring_status;
}  // namespace

// Device address of g_ring_status on the current device (looked up once per device), or nullptr.
int* ring_status_word() {
    static int* addr[64] = {};
    static std::mutex m;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        set_error("no current CUDA device");
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(m);
    if (!addr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_ring_status);
        if (e != cudaSuccess) {
            cuda_fail(e, "cudaGetSymbolAddress(status word)");
            return nullptr;
        }
        addr[dev] = static_cast<int*>(p);
    }
    return addr[dev];
}

int launch_fc_decode_ring(const float* x, int rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng, int64_t Kg,
                          int qtype, int G, int64_t N, float* y, int64_t ldy, unsigned flags, cudaStream_t s, void* ws,
                          size_t ws_bytes, const void* xq, const float* addend, int64_t addend_ld) {
    const RingCall c = {x, ldx, xq, rows, K, Kg, wq, Ng, N, y, ldy, addend, addend_ld};
    return launch_ring_impl<false>(&c, 1, qtype, G, flags, s, nullptr, ws, ws_bytes);
}

int launch_fc_decode_ring_multi(const float* x, int rows, int64_t K, int64_t ldx, int64_t Kg, int qtype, int G,
                                const q4fc_fc_job* jobs, int njobs, unsigned flags, cudaStream_t s, void* ws,
                                size_t ws_bytes, const void* xq) {
    RingCall c[kMaxJobs];
    for (int i = 0; i < njobs; i++)
        c[i] = {x, ldx, xq, rows, K, Kg, static_cast<const uint8_t*>(jobs[i].wq), jobs[i].Ng, jobs[i].N, jobs[i].y,
                jobs[i].ldy, jobs[i].addend, jobs[i].ld_addend};
    return launch_ring_impl<false>(c, njobs, qtype, G, flags, s, nullptr, ws, ws_bytes);
}

int launch_fc_decode_ring_batch(const q4fc_fc_call* calls, int ncalls, int qtype, int G, unsigned flags,
                                cudaStream_t s) {
    RingCall c[kMaxJobs];
    for (int i = 0; i < ncalls; i++)
        c[i] = {nullptr, 0, calls[i].xq, (int)calls[i].rows, calls[i].K, calls[i].Kg,
                static_cast<const uint8_t*>(calls[i].wq), calls[i].Ng, calls[i].N, calls[i].y, calls[i].ldy,
                calls[i].addend, calls[i].ld_addend};
    return launch_ring_impl<false>(c, ncalls, qtype, G, flags, s, nullptr, nullptr, 0);
}

}  // namespace q4fc
