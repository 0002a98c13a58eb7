// Shared definitions of the sm_100a quantized-FC kernels: the reference's
// block layout (ops/op_fc.hpp:14-24, 64-71), error plumbing and small device
// helpers.  One block = 32 columns x G k:
//   bytes [0, 16*G)           G/8 rows of 128 B; a 32-bit word at row r,
//                             column n holds k = 8r..8r+3 in the low nibbles
//                             of its 4 bytes and k = 8r+4..8r+7 in the high
//   bytes [16*G, 16*G+64)     32 fp16 scales wd
//   bytes [16*G+64, +128)     32 fp16 minima wm (Q4_1 only)
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/q4fc_b200.h"

namespace q4fc {

constexpr int kGroupN = 32;  // columns per block (group_n, ops/op_fc.hpp:17)
constexpr int kMaxDecodeRows = 8;

__host__ __device__ constexpr int block_bytes(int qtype, int G) { return 16 * G + (qtype ? 128 : 64); }

inline bool valid_variant(int qtype, int G) { return (qtype == 0 || qtype == 1) && (G == 32 || G == 128); }

// thread-local detail text behind q4fc_last_error()
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define Q4FC_CUDA_OK(expr)                                     \
    do {                                                       \
        cudaError_t e__ = (expr);                              \
        if (e__ != cudaSuccess) return q4fc::cuda_fail(e__, #expr); \
    } while (0)

struct DeviceInfo {
    int sm_count;
    int max_smem_optin;
};
// cached per device; returns nullptr (and sets the error text) on failure
const DeviceInfo* device_info();

// ---- workspace layout of the FC entry points ------------------------------
// [0, 256)   status word (int) + padding
// then       CTA partials [ctas][2][8][32] fp32 (size fixed per device)
// then       per-stripe arrival counters int[Ng], zero between calls
constexpr size_t kWsStatusBytes = 256;

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// launchers implemented in the kernel translation units
int launch_pack(const float* w, int64_t N, int64_t K, int qtype, int G, uint8_t* wq, cudaStream_t s);
int launch_dequant(const uint8_t* wq, int64_t Ng, int64_t Kg, int qtype, int G, int nibble_signed, float* out,
                   cudaStream_t s);
int launch_quant_x(const float* x, int64_t rows, int64_t K, int64_t ldx, int G, float scale, int8_t* codes,
                   float* scales, float* gsums, cudaStream_t s);
constexpr size_t kWsCounterCapacity = 64 * 1024;  // stripe counters of N <= 524288 end before the quantizer scratch
size_t decode_workspace_bytes(int64_t N);
size_t decode_prequant_offset();
int launch_fc_decode(const float* x, int rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng, int64_t Kg,
                     int qtype, int G, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes, unsigned flags,
                     cudaStream_t s);
// ring form of the decode kernel (bulk copies into a shared-memory ring; no global scratch): fc_decode_ring*.cu
int launch_fc_decode_ring(const float* x, int rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng, int64_t Kg,
                          int qtype, int G, int64_t N, float* y, int64_t ldy, unsigned flags, cudaStream_t s,
                          void* ws = nullptr, size_t ws_bytes = 0, const void* xq = nullptr,
                          const float* addend = nullptr, int64_t addend_ld = 0);
// several weight tensors on one input in one launch
int launch_fc_decode_ring_multi(const float* x, int rows, int64_t K, int64_t ldx, int64_t Kg, int qtype, int G,
                                const q4fc_fc_job* jobs, int njobs, unsigned flags, cudaStream_t s, void* ws,
                                size_t ws_bytes, const void* xq);
// a batch of independent FCs on pre-quantized inputs in one launch
int launch_fc_decode_ring_batch(const q4fc_fc_call* calls, int ncalls, int qtype, int G, unsigned flags, cudaStream_t s);
// device address of the status word used by launches without a workspace (current device), or nullptr
int* ring_status_word();
// RMS normalization fused with the quantizer (rmsnorm_quant.cu); writes the pre-quantized format
int launch_rmsnorm_quant(const float* x, const float* residual, float* sum_out, int rows, int64_t K, int64_t ldx,
                         const float* weight, float eps, float* y,
                         int64_t ldy, int G, bool want_isum, int8_t* codes, float* sc, bool pdl, cudaStream_t s);
// quantizing launch in front of the decode FC for large rows x K (scratch layout: quant_x.cu)
size_t quant_pre_bytes(int64_t rows, int64_t K, int G);
// `up` != nullptr: quantize silu(x) * up instead of x (rows of `up` share x's stride); `prod`: optional fp32 copy
int launch_quant_x_pre(const float* x, int rows, int64_t K, int64_t ldx, int G, bool want_isum, int8_t* codes,
                       float* sc, bool pdl, cudaStream_t s, const float* up = nullptr, float* prod = nullptr,
                       int64_t ldp = 0);
int launch_quant_x_pre_batch(const q4fc_xq_call* calls, int n, int G, bool want_isum, bool pdl, cudaStream_t s);
// the same kernel with outputs stored, epoch-stamped, into every rank's buffer (tp->y_peer)
int launch_fc_decode_ring_tp(const float* x, int rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng,
                                int64_t Kg, int qtype, int G, int64_t N, int64_t ldy, unsigned flags, cudaStream_t s,
                                const q4fc_tp_site* tp);
int launch_fc_decode_ring_tp_batch(const q4fc_tp_call* calls, const q4fc_tp_site* const* sites, int ncalls, int qtype,
                                   int G, unsigned flags, cudaStream_t s);
int launch_tp_collect_multi(const unsigned long long* const* src, const int64_t* rows, const int64_t* N,
                            const int64_t* ld, float* const* dst, const int64_t* ldd, int n,
                            const unsigned long long* epoch, int* status, cudaStream_t s);
// step barrier and stream-side wait of the N-split over several GPUs
int launch_tp_step_begin(unsigned long long* epoch, unsigned long long* const* barrier_peer,
                         const unsigned long long* barrier_local, int world, int* status, cudaStream_t s);
int launch_tp_collect(const unsigned long long* src, int64_t rows, int64_t N, int64_t ld, float* dst, int64_t ldd,
                      const unsigned long long* epoch, int* status, cudaStream_t s);
// per-channel int8 weights and the quantized embedding table (q8c.cu)
int launch_q8c_pack(const float* w, int64_t N, int64_t K, int8_t* wq, float* wscales, cudaStream_t s);
size_t q8c_workspace_bytes(int64_t rows, int64_t K);
int launch_q8c_fc(const float* x, int64_t rows, int64_t K, int64_t ldx, const int8_t* wq, const float* wscales,
                  int64_t Ng, int64_t Kg, int64_t N, float* y, int64_t ldy, void* ws, cudaStream_t s);
int launch_emb_q8c_quant(const float* table, int64_t V, int64_t E, int8_t* codes, float* scales, cudaStream_t s);
int launch_emb_q8c(const void* ids, int ids_are_i32, int64_t n, const int8_t* codes, const float* scales, int64_t V,
                   int64_t E, float* out, int64_t ldo, cudaStream_t s);
// a chain of dependent decode FCs as one persistent launch (fc_chain.cu)
int chain_create(const q4fc_chain_step* steps, int nsteps, const q4fc_fc_job* jobs, int njobs, int rows, int qtype, int G,
                 void** out);
int chain_run(void* chain, cudaStream_t s);
int chain_check(void* chain, cudaStream_t s);
int chain_destroy(void* chain);
size_t prefill_workspace_bytes(int64_t rows, int64_t K, int64_t N, int qtype, int G);
int launch_fc_prefill(const float* x, int64_t rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng,
                      int64_t Kg, int qtype, int G, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes,
                      unsigned flags, cudaStream_t s);

#ifdef __CUDACC__
__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t f2h_rn(float f) { return __half_as_ushort(__float2half_rn(f)); }

// x / y for a constant y in {7, 15, 127} and x >= 0, correctly rounded like the IEEE division the
// reference performs, without the division sequence: q = x*c, r = fma(-y, q, x), q' = fma(r, c, q) with
// c = fl(1/y).  Checked exhaustively on the host against x / y for every non-negative finite fp32 x
// (all three constants): no mismatch.  Infinite / NaN x fall through to q.
__device__ __forceinline__ float div_const_rn(float x, float y, float c) {
    const float q = __fmul_rn(x, c);
    const float r = __fmaf_rn(-y, q, x);
    const float q2 = __fmaf_rn(r, c, q);
    return (r == r) ? q2 : q;
}
// 1 / d as the reference computes it (IEEE division), 0 for d == 0
__device__ __forceinline__ float inv_or_zero(float d) { return (d != 0.0f) ? __frcp_rn(d) : 0.0f; }

// streaming 128-bit load: read-only path, no L1 allocation
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream_v2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// programmatic dependent launch: both are no-ops when the kernel was launched
// without the programmatic-serialization attribute
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

}  // namespace q4fc
