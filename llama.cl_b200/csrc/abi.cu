// extern "C" entry points declared in include/q4fc_b200.h: argument checks,
// error text, dispatch to the kernel launchers.  No entry point allocates or
// synchronizes (q4fc_fc_check_status excepted, which is documented as
// host-synchronous).
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace q4fc {

namespace {
thread_local char g_err[512] = "";
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
    return Q4FC_ECUDA;
}

const DeviceInfo* device_info() {
    static DeviceInfo info[64];
    static bool ready[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        set_error("no current CUDA device");
        return nullptr;
    }
    static std::mutex m;  // first calls on a device may come from several host threads
    std::lock_guard<std::mutex> lk(m);
    if (!ready[dev]) {
        int sms = 0, smem = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
            cudaGetLastError();
            set_error("cannot query device %d", dev);
            return nullptr;
        }
        info[dev].sm_count = sms;
        info[dev].max_smem_optin = smem;
        ready[dev] = true;
    }
    return &info[dev];
}

namespace {

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

int check_variant(int qtype, int G, const char* who) {
    if (!valid_variant(qtype, G)) {
        set_error("%s: unsupported block type (qtype=%d, group_k=%d); expected Q4_0/Q4_1 with group 32 or 128", who,
                  qtype, G);
        return Q4FC_EVARIANT;
    }
    return Q4FC_OK;
}

int check_fc_args(const char* who, const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng,
                  int64_t Kg, int qtype, int G, int64_t N, float* y, int64_t ldy) {
    if (int rc = check_variant(qtype, G, who)) return rc;
    if (rows < 0 || K <= 0 || N < 0 || Ng < 0 || Kg <= 0) {
        set_error("%s: negative or empty size (rows=%lld K=%lld N=%lld Ng=%lld Kg=%lld)", who, (long long)rows,
                  (long long)K, (long long)N, (long long)Ng, (long long)Kg);
        return Q4FC_EINVAL;
    }
    if ((K + G - 1) / G != Kg) {
        set_error("%s: K=%lld does not match Kg=%lld groups of %d", who, (long long)K, (long long)Kg, G);
        return Q4FC_EINVAL;
    }
    if (N > Ng * 32) {
        set_error("%s: N=%lld exceeds the %lld columns of the packed tensor", who, (long long)N, (long long)(Ng * 32));
        return Q4FC_EINVAL;
    }
    if (rows > 0 && N > 0) {
        if (!x || !wq || !y) {
            set_error("%s: null pointer", who);
            return Q4FC_EINVAL;
        }
        if (ldx < K || ldy < N) {
            set_error("%s: leading dimension smaller than the row (ldx=%lld K=%lld ldy=%lld N=%lld)", who,
                      (long long)ldx, (long long)K, (long long)ldy, (long long)N);
            return Q4FC_EINVAL;
        }
        if (!aligned(wq, 16) || !aligned(x, 4) || !aligned(y, 4)) {
            set_error("%s: packed weights need 16-byte alignment, x and y 4-byte", who);
            return Q4FC_EALIGN;
        }
    }
    return Q4FC_OK;
}

}  // namespace
}  // namespace q4fc

using namespace q4fc;

extern "C" {

int q4fc_version(void) { return 100; }

const char* q4fc_strerror(int code) {
    switch (code) {
        case Q4FC_OK: return "ok";
        case Q4FC_EINVAL: return "invalid argument";
        case Q4FC_EVARIANT: return "unsupported block variant";
        case Q4FC_EALIGN: return "misaligned pointer or leading dimension";
        case Q4FC_EWORKSPACE: return "workspace missing or too small";
        case Q4FC_ECUDA: return "CUDA runtime error";
        case Q4FC_EDEVICE: return "device-side wait ran out";
        case Q4FC_ELIMIT: return "size beyond a supported maximum";
        default: return "unknown error";
    }
}

const char* q4fc_last_error(void) { return g_err; }

int q4fc_block_bytes(int qtype, int group_k) { return valid_variant(qtype, group_k) ? block_bytes(qtype, group_k) : -1; }

int q4fc_infer_variant(int bs, int* qtype, int* group_k) {
    for (int q = 0; q < 2; q++)
        for (int G : {32, 128})
            if (block_bytes(q, G) == bs) {
                if (qtype) *qtype = q;
                if (group_k) *group_k = G;
                return Q4FC_OK;
            }
    set_error("block size %d is none of 576 / 640 / 2112 / 2176", bs);
    return Q4FC_EVARIANT;
}

int q4fc_pack(const float* w, int64_t N, int64_t K, int qtype, int group_k, void* wq, q4fc_stream_t stream) {
    if (int rc = check_variant(qtype, group_k, "pack")) return rc;
    if (N < 0 || K < 0) {
        set_error("pack: negative size");
        return Q4FC_EINVAL;
    }
    if (N == 0 || K == 0) return Q4FC_OK;
    if (!w || !wq) {
        set_error("pack: null pointer");
        return Q4FC_EINVAL;
    }
    if (!aligned(wq, 16) || !aligned(w, 4)) {
        set_error("pack: output needs 16-byte alignment, input 4-byte");
        return Q4FC_EALIGN;
    }
    return launch_pack(w, N, K, qtype, group_k, static_cast<uint8_t*>(wq), static_cast<cudaStream_t>(stream));
}

int q4fc_dequant(const void* wq, int64_t Ng, int64_t Kg, int qtype, int group_k, int nibble_signed, float* out,
                 q4fc_stream_t stream) {
    if (int rc = check_variant(qtype, group_k, "dequant")) return rc;
    if (Ng < 0 || Kg < 0) {
        set_error("dequant: negative size");
        return Q4FC_EINVAL;
    }
    if (Ng == 0 || Kg == 0) return Q4FC_OK;
    if (!wq || !out) {
        set_error("dequant: null pointer");
        return Q4FC_EINVAL;
    }
    if (!aligned(wq, 4) || !aligned(out, 16)) {
        set_error("dequant: output needs 16-byte alignment, packed input 4-byte");
        return Q4FC_EALIGN;
    }
    return launch_dequant(static_cast<const uint8_t*>(wq), Ng, Kg, qtype, group_k, nibble_signed, out,
                          static_cast<cudaStream_t>(stream));
}

int q4fc_quant_x(const float* x, int64_t rows, int64_t K, int64_t ldx, int group_k, float scale, int8_t* codes,
                 float* scales, float* gsums, q4fc_stream_t stream) {
    if (group_k != 32 && group_k != 128) {
        set_error("quant_x: group_k=%d, expected 32 or 128", group_k);
        return Q4FC_EVARIANT;
    }
    if (rows < 0 || K < 0) {
        set_error("quant_x: negative size");
        return Q4FC_EINVAL;
    }
    if (rows == 0 || K == 0) return Q4FC_OK;
    if (!x || !codes || !scales) {
        set_error("quant_x: null pointer");
        return Q4FC_EINVAL;
    }
    if (ldx < K) {
        set_error("quant_x: ldx=%lld smaller than K=%lld", (long long)ldx, (long long)K);
        return Q4FC_EINVAL;
    }
    if (!aligned(codes, 4) || !aligned(x, 4)) {
        set_error("quant_x: codes and x need 4-byte alignment");
        return Q4FC_EALIGN;
    }
    return launch_quant_x(x, rows, K, ldx, group_k, scale, codes, scales, gsums, static_cast<cudaStream_t>(stream));
}

size_t q4fc_fc_workspace_bytes(int64_t rows, int64_t K, int64_t N, int qtype, int group_k) {
    if (!valid_variant(qtype, group_k) || rows < 0 || K < 0 || N < 0) return 0;
    size_t need = decode_workspace_bytes((N + 31) / 32 * 32);
    if (rows <= kMaxDecodeRows) {  // room for the quantizing launch in front of the decode kernel
        const size_t q = decode_prequant_offset() + quant_pre_bytes(rows, K, group_k);
        if (q > need) need = q;
    }
    if (rows > kMaxDecodeRows) {
        size_t p = prefill_workspace_bytes(rows, K, N, qtype, group_k);
        if (p > need) need = p;
    }
    return need;
}

int q4fc_fc_workspace_init(void* ws, size_t ws_bytes, q4fc_stream_t stream) {
    if (!ws || ws_bytes < kWsStatusBytes) {
        set_error("workspace_init: null or tiny workspace");
        return Q4FC_EWORKSPACE;
    }
    if (!aligned(ws, 256)) {
        set_error("workspace_init: workspace needs 256-byte alignment");
        return Q4FC_EALIGN;
    }
    Q4FC_CUDA_OK(cudaMemsetAsync(ws, 0, ws_bytes, static_cast<cudaStream_t>(stream)));
    return Q4FC_OK;
}

int q4fc_fc_decode(const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg,
                   int qtype, int group_k, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes,
                   unsigned flags, q4fc_stream_t stream) {
    if (int rc = check_fc_args("fc_decode", x, rows, K, ldx, wq, Ng, Kg, qtype, group_k, N, y, ldy)) return rc;
    if (rows > kMaxDecodeRows) {
        set_error("fc_decode: rows=%lld exceeds %d; use q4fc_fc or q4fc_fc_prefill", (long long)rows, kMaxDecodeRows);
        return Q4FC_ELIMIT;
    }
    if (ws && !aligned(ws, 256)) {
        set_error("fc_decode: workspace needs 256-byte alignment");
        return Q4FC_EALIGN;
    }
    if (flags & Q4FC_FLAG_STREAMK)
        return launch_fc_decode(x, (int)rows, K, ldx, static_cast<const uint8_t*>(wq), Ng, Kg, qtype, group_k, N, y,
                                ldy, ws, ws_bytes, flags, static_cast<cudaStream_t>(stream));
    return launch_fc_decode_ring(x, (int)rows, K, ldx, static_cast<const uint8_t*>(wq), Ng, Kg, qtype, group_k, N,
                                    y, ldy, flags, static_cast<cudaStream_t>(stream), ws, ws_bytes);
}

size_t q4fc_xq_bytes(int64_t rows, int64_t K, int group_k) {
    if ((group_k != 32 && group_k != 128) || rows < 0 || K < 0) return 0;
    return quant_pre_bytes(rows, K, group_k);
}

static int check_xq_args(const char* who, int64_t rows, int64_t K, int group_k, const void* xq) {
    if (group_k != 32 && group_k != 128) {
        set_error("%s: group_k=%d is neither 32 nor 128", who, group_k);
        return Q4FC_EVARIANT;
    }
    if (rows < 0 || rows > kMaxDecodeRows || K <= 0) {
        set_error("%s: rows=%lld must be 0..%d and K=%lld positive", who, (long long)rows, kMaxDecodeRows, (long long)K);
        return rows > kMaxDecodeRows ? Q4FC_ELIMIT : Q4FC_EINVAL;
    }
    if (rows > 0 && (!xq || !aligned(xq, 256))) {
        set_error("%s: xq is null or not 256-byte aligned", who);
        return xq ? Q4FC_EALIGN : Q4FC_EINVAL;
    }
    return Q4FC_OK;
}

int q4fc_quant_x_q8(const float* x, int64_t rows, int64_t K, int64_t ldx, int group_k, int want_isum, void* xq,
                    unsigned flags, q4fc_stream_t stream) {
    if (int rc = check_xq_args("quant_x_q8", rows, K, group_k, xq)) return rc;
    if (rows == 0) return Q4FC_OK;
    if (!x || ldx < K || !aligned(x, 4)) {
        set_error("quant_x_q8: null or misaligned x, or ldx < K");
        return Q4FC_EINVAL;
    }
    const int64_t Kg = (K + group_k - 1) / group_k;
    uint8_t* base = static_cast<uint8_t*>(xq);
    return launch_quant_x_pre(x, (int)rows, K, ldx, group_k, want_isum != 0, reinterpret_cast<int8_t*>(base),
                              reinterpret_cast<float*>(base + align_up((size_t)(rows * Kg * group_k), 256)),
                              (flags & Q4FC_FLAG_PDL) != 0, static_cast<cudaStream_t>(stream));
}

int q4fc_quant_x_q8_batch(const q4fc_xq_call* calls, int ncalls, int group_k, int want_isum, unsigned flags,
                          q4fc_stream_t stream) {
    if (ncalls < 0 || ncalls > 16 || (ncalls > 0 && !calls)) {
        set_error("quant_x_q8_batch: ncalls=%d outside 0..16, or null calls", ncalls);
        return Q4FC_ELIMIT;
    }
    for (int i = 0; i < ncalls; i++) {
        const q4fc_xq_call& c = calls[i];
        if (int rc = check_xq_args("quant_x_q8_batch", c.rows, c.K, group_k, c.xq)) return rc;
        if (c.rows > 0 && (!c.x || c.ldx < c.K || !aligned(c.x, 4))) {
            set_error("quant_x_q8_batch: call %d: null or misaligned x, or ldx < K", i);
            return Q4FC_EINVAL;
        }
    }
    return launch_quant_x_pre_batch(calls, ncalls, group_k, want_isum != 0, (flags & Q4FC_FLAG_PDL) != 0,
                                    static_cast<cudaStream_t>(stream));
}

int q4fc_silu_mul_quant(const float* gate, const float* up, int64_t rows, int64_t K, int64_t ld, float* prod, int64_t ldp,
                        int group_k, int want_isum, void* xq, unsigned flags, q4fc_stream_t stream) {
    if (int rc = check_xq_args("silu_mul_quant", rows, K, group_k, xq)) return rc;
    if (rows == 0) return Q4FC_OK;
    if (!gate || !up || ld < K || !aligned(gate, 4) || !aligned(up, 4) || (prod && (ldp < K || !aligned(prod, 4)))) {
        set_error("silu_mul_quant: null or misaligned gate / up / prod, or a leading dimension smaller than K");
        return Q4FC_EINVAL;
    }
    const int64_t Kg = (K + group_k - 1) / group_k;
    uint8_t* base = static_cast<uint8_t*>(xq);
    return launch_quant_x_pre(gate, (int)rows, K, ld, group_k, want_isum != 0, reinterpret_cast<int8_t*>(base),
                              reinterpret_cast<float*>(base + align_up((size_t)(rows * Kg * group_k), 256)),
                              (flags & Q4FC_FLAG_PDL) != 0, static_cast<cudaStream_t>(stream), up, prod, ldp);
}

int q4fc_rmsnorm_quant(const float* x, int64_t rows, int64_t K, int64_t ldx, const float* weight, float eps, float* y,
                       int64_t ldy, int group_k, int want_isum, void* xq, unsigned flags, q4fc_stream_t stream) {
    return q4fc_add_rmsnorm_quant(x, nullptr, nullptr, rows, K, ldx, weight, eps, y, ldy, group_k, want_isum, xq,
                                  flags, stream);
}

int q4fc_add_rmsnorm_quant(const float* x, const float* residual, float* sum_out, int64_t rows, int64_t K, int64_t ldx,
                           const float* weight, float eps, float* y, int64_t ldy, int group_k, int want_isum,
                           void* xq, unsigned flags, q4fc_stream_t stream) {
    if (int rc = check_xq_args("rmsnorm_quant", rows, K, group_k, xq)) return rc;
    if (sum_out && !residual) {
        set_error("rmsnorm_quant: sum_out without residual");
        return Q4FC_EINVAL;
    }
    if ((residual && !aligned(residual, 16)) || (sum_out && !aligned(sum_out, 16))) {
        set_error("rmsnorm_quant: residual and sum_out need 16-byte alignment");
        return Q4FC_EALIGN;
    }
    if (rows == 0) return Q4FC_OK;
    if (K % 8 != 0) {
        set_error("rmsnorm_quant: K=%lld must be a multiple of 8 (as in the reference)", (long long)K);
        return Q4FC_EINVAL;
    }
    if (!x || !weight || ldx < K || (y && ldy < K)) {
        set_error("rmsnorm_quant: null pointer or leading dimension smaller than K");
        return Q4FC_EINVAL;
    }
    if (!aligned(x, 16) || !aligned(weight, 16) || (y && !aligned(y, 16)) || ldx % 4 != 0 || (y && ldy % 4 != 0)) {
        set_error("rmsnorm_quant: x, weight and y need 16-byte alignment and leading dimensions divisible by 4");
        return Q4FC_EALIGN;
    }
    const int64_t Kg = (K + group_k - 1) / group_k;
    uint8_t* base = static_cast<uint8_t*>(xq);
    return launch_rmsnorm_quant(x, residual, sum_out, (int)rows, K, ldx, weight, eps, y, ldy, group_k, want_isum != 0,
                                reinterpret_cast<int8_t*>(base),
                                reinterpret_cast<float*>(base + align_up((size_t)(rows * Kg * group_k), 256)),
                                (flags & Q4FC_FLAG_PDL) != 0, static_cast<cudaStream_t>(stream));
}

int q4fc_fc_decode_q8(const void* xq, int64_t rows, int64_t K, const void* wq, int64_t Ng, int64_t Kg, int qtype,
                      int group_k, int64_t N, float* y, int64_t ldy, unsigned flags, q4fc_stream_t stream) {
    if (int rc = check_xq_args("fc_decode_q8", rows, K, group_k, xq)) return rc;
    // the codes stand in for x in the shared argument checks (pointer non-null, 4-byte aligned)
    if (int rc = check_fc_args("fc_decode_q8", static_cast<const float*>(xq), rows, K, K, wq, Ng, Kg, qtype, group_k, N,
                               y, ldy))
        return rc;
    if (flags & Q4FC_FLAG_STREAMK) {
        set_error("fc_decode_q8: Q4FC_FLAG_STREAMK is not available for pre-quantized activations");
        return Q4FC_EINVAL;
    }
    return launch_fc_decode_ring(nullptr, (int)rows, K, K, static_cast<const uint8_t*>(wq), Ng, Kg, qtype, group_k,
                                    N, y, ldy, flags, static_cast<cudaStream_t>(stream), nullptr, 0, xq);
}

int q4fc_fc_decode_add(const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg,
                       int qtype, int group_k, int64_t N, float* y, int64_t ldy, const float* addend,
                       int64_t ld_addend, void* ws, size_t ws_bytes, unsigned flags, q4fc_stream_t stream) {
    if (int rc = check_fc_args("fc_decode_add", x, rows, K, ldx, wq, Ng, Kg, qtype, group_k, N, y, ldy)) return rc;
    if (rows > kMaxDecodeRows) {
        set_error("fc_decode_add: rows=%lld exceeds %d", (long long)rows, kMaxDecodeRows);
        return Q4FC_ELIMIT;
    }
    if (flags & Q4FC_FLAG_STREAMK) {
        set_error("fc_decode_add: Q4FC_FLAG_STREAMK is not available with an addend");
        return Q4FC_EINVAL;
    }
    if (rows > 0 && N > 0 && (!addend || !aligned(addend, 4) || ld_addend < 0 || (ld_addend != 0 && ld_addend < N))) {
        set_error("fc_decode_add: addend is null or misaligned, or 0 < ld_addend < N");
        return Q4FC_EINVAL;
    }
    if (ws && !aligned(ws, 256)) {
        set_error("fc_decode_add: workspace needs 256-byte alignment");
        return Q4FC_EALIGN;
    }
    return launch_fc_decode_ring(x, (int)rows, K, ldx, static_cast<const uint8_t*>(wq), Ng, Kg, qtype, group_k, N,
                                    y, ldy, flags, static_cast<cudaStream_t>(stream), ws, ws_bytes, nullptr, addend,
                                    ld_addend);
}

int q4fc_fc_decode_multi(const float* x, const void* xq, int64_t rows, int64_t K, int64_t ldx, int64_t Kg, int qtype,
                         int group_k, const q4fc_fc_job* jobs, int njobs, void* ws, size_t ws_bytes, unsigned flags,
                         q4fc_stream_t stream) {
    if (!jobs || njobs < 1 || njobs > 4) {
        set_error("fc_decode_multi: null jobs or njobs=%d outside 1..4", njobs);
        return Q4FC_EINVAL;
    }
    if ((x == nullptr) == (xq == nullptr)) {
        set_error("fc_decode_multi: exactly one of x and xq must be given");
        return Q4FC_EINVAL;
    }
    if (xq) {
        if (int rc = check_xq_args("fc_decode_multi", rows, K, group_k, xq)) return rc;
        ldx = K;
    }
    if (rows > kMaxDecodeRows) {
        set_error("fc_decode_multi: rows=%lld exceeds %d", (long long)rows, kMaxDecodeRows);
        return Q4FC_ELIMIT;
    }
    if (flags & Q4FC_FLAG_STREAMK) {
        set_error("fc_decode_multi: Q4FC_FLAG_STREAMK is not available for several weight tensors");
        return Q4FC_EINVAL;
    }
    if (ws && !aligned(ws, 256)) {
        set_error("fc_decode_multi: workspace needs 256-byte alignment");
        return Q4FC_EALIGN;
    }
    for (int i = 0; i < njobs; i++) {
        const q4fc_fc_job& jb = jobs[i];
        // with codes as input they stand in for x in the shared argument checks (pointer non-null, 4-byte aligned)
        if (int rc = check_fc_args("fc_decode_multi", x ? x : static_cast<const float*>(xq), rows, K, ldx, jb.wq, jb.Ng,
                                   Kg, qtype, group_k, jb.N, jb.y, jb.ldy))
            return rc;
        if (rows > 0 && jb.N > 0 && jb.addend &&
            (!aligned(jb.addend, 4) || jb.ld_addend < 0 || (jb.ld_addend != 0 && jb.ld_addend < jb.N))) {
            set_error("fc_decode_multi: job %d: addend is misaligned, or 0 < ld_addend < N", i);
            return Q4FC_EINVAL;
        }
    }
    return launch_fc_decode_ring_multi(x, (int)rows, K, ldx, Kg, qtype, group_k, jobs, njobs, flags,
                                       static_cast<cudaStream_t>(stream), ws, ws_bytes, xq);
}

int q4fc_fc_decode_batch(const q4fc_fc_call* calls, int ncalls, int qtype, int group_k, unsigned flags,
                         q4fc_stream_t stream) {
    if (!calls || ncalls < 1 || ncalls > 16) {
        set_error("fc_decode_batch: null calls or ncalls=%d outside 1..16", ncalls);
        return Q4FC_EINVAL;
    }
    if (flags & Q4FC_FLAG_STREAMK) {
        set_error("fc_decode_batch: Q4FC_FLAG_STREAMK is not available for a batch");
        return Q4FC_EINVAL;
    }
    for (int i = 0; i < ncalls; i++) {
        const q4fc_fc_call& c = calls[i];
        if (int rc = check_xq_args("fc_decode_batch", c.rows, c.K, group_k, c.xq)) return rc;
        if (int rc = check_fc_args("fc_decode_batch", static_cast<const float*>(c.xq), c.rows, c.K, c.K, c.wq, c.Ng, c.Kg,
                                   qtype, group_k, c.N, c.y, c.ldy))
            return rc;
        if (c.rows > 0 && c.N > 0 && c.addend &&
            (!aligned(c.addend, 4) || c.ld_addend < 0 || (c.ld_addend != 0 && c.ld_addend < c.N))) {
            set_error("fc_decode_batch: call %d: addend is misaligned, or 0 < ld_addend < N", i);
            return Q4FC_EINVAL;
        }
    }
    return launch_fc_decode_ring_batch(calls, ncalls, qtype, group_k, flags, static_cast<cudaStream_t>(stream));
}

int q4fc_fc_prefill(const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg,
                    int qtype, int group_k, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes,
                    unsigned flags, q4fc_stream_t stream) {
    if (int rc = check_fc_args("fc_prefill", x, rows, K, ldx, wq, Ng, Kg, qtype, group_k, N, y, ldy)) return rc;
    if (ws && !aligned(ws, 256)) {
        set_error("fc_prefill: workspace needs 256-byte alignment");
        return Q4FC_EALIGN;
    }
    return launch_fc_prefill(x, rows, K, ldx, static_cast<const uint8_t*>(wq), Ng, Kg, qtype, group_k, N, y, ldy, ws,
                             ws_bytes, flags, static_cast<cudaStream_t>(stream));
}

int q4fc_fc(const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg, int qtype,
            int group_k, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes, unsigned flags,
            q4fc_stream_t stream) {
    if (rows <= kMaxDecodeRows)
        return q4fc_fc_decode(x, rows, K, ldx, wq, Ng, Kg, qtype, group_k, N, y, ldy, ws, ws_bytes, flags, stream);
    return q4fc_fc_prefill(x, rows, K, ldx, wq, Ng, Kg, qtype, group_k, N, y, ldy, ws, ws_bytes, flags, stream);
}

size_t q4fc_tp_site_bytes(void) { return sizeof(q4fc_tp_site); }

int q4fc_tp_arena_create(size_t bytes, void** base, void* ipc_handle_64) {
    if (!base || !ipc_handle_64 || bytes == 0) {
        set_error("tp_arena_create: null argument or zero size");
        return Q4FC_EINVAL;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the IPC handle is shipped as 64 bytes");
    void* p = nullptr;
    Q4FC_CUDA_OK(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return cuda_fail(e, "tp_arena_create");
    }
    memcpy(ipc_handle_64, &h, sizeof(h));
    *base = p;
    return Q4FC_OK;
}

int q4fc_tp_arena_open(const void* ipc_handle_64, void** peer_base) {
    if (!ipc_handle_64 || !peer_base) {
        set_error("tp_arena_open: null argument");
        return Q4FC_EINVAL;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle_64, sizeof(h));
    Q4FC_CUDA_OK(cudaIpcOpenMemHandle(peer_base, h, cudaIpcMemLazyEnablePeerAccess));
    return Q4FC_OK;
}

int q4fc_tp_arena_close(void* peer_base) {
    if (peer_base) Q4FC_CUDA_OK(cudaIpcCloseMemHandle(peer_base));
    return Q4FC_OK;
}

int q4fc_tp_arena_destroy(void* base) {
    if (base) Q4FC_CUDA_OK(cudaFree(base));
    return Q4FC_OK;
}

int q4fc_tp_step_begin(unsigned long long* epoch, unsigned long long* const* barrier_peer,
                       const unsigned long long* barrier_local, int world, int* status, q4fc_stream_t stream) {
    if (!epoch || !barrier_peer || !barrier_local || !status || world < 1 || world > 8) {
        set_error("tp_step_begin: null argument or world=%d outside 1..8", world);
        return Q4FC_EINVAL;
    }
    for (int i = 0; i < world; i++)
        if (!barrier_peer[i] || !aligned(barrier_peer[i], 8)) {
            set_error("tp_step_begin: barrier_peer[%d] is null or misaligned", i);
            return Q4FC_EINVAL;
        }
    return launch_tp_step_begin(epoch, barrier_peer, barrier_local, world, status, static_cast<cudaStream_t>(stream));
}

int q4fc_tp_collect(const unsigned long long* stamped, int64_t rows, int64_t N, int64_t ld, float* dst, int64_t ldd,
                    const unsigned long long* epoch, int* status, q4fc_stream_t stream) {
    if (!stamped || !dst || !epoch || !status || rows < 0 || N < 0 || ld < N || ldd < N || !aligned(stamped, 8)) {
        set_error("tp_collect: null or misaligned pointer, negative size, or pitch smaller than N");
        return Q4FC_EINVAL;
    }
    return launch_tp_collect(stamped, rows, N, ld, dst, ldd, epoch, status, static_cast<cudaStream_t>(stream));
}

int q4fc_fc_decode_tp(const void* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg,
                      int qtype, int group_k, int64_t N, int64_t ldy, const q4fc_tp_site* site, unsigned flags,
                      q4fc_stream_t stream) {
    if (!site || site->world < 1 || site->world > 8 || !site->epoch || !site->status) {
        set_error("fc_decode_tp: null site, or world outside 1..8, or null epoch/status");
        return Q4FC_EINVAL;
    }
    if (flags & Q4FC_FLAG_STREAMK) {
        set_error("fc_decode_tp: Q4FC_FLAG_STREAMK is not available for the multi-GPU form");
        return Q4FC_EINVAL;
    }
    if (site->col_off < 0 || site->col_off % 32 != 0 || site->col_off + N > ldy) {
        set_error("fc_decode_tp: col_off=%lld must be a multiple of 32 with col_off + N <= ldy",
                  (long long)site->col_off);
        return Q4FC_EINVAL;
    }
    for (int i = 0; i < site->world; i++)
        if (!site->y_peer[i] || !aligned(site->y_peer[i], 8)) {
            set_error("fc_decode_tp: y_peer[%d] is null or not 8-byte aligned", i);
            return Q4FC_EINVAL;
        }
    if (site->xq_scratch && !aligned(site->xq_scratch, 256)) {
        set_error("fc_decode_tp: xq_scratch needs 256-byte alignment");
        return Q4FC_EALIGN;
    }
    if (site->x_stamped && !aligned(x, 8)) {
        set_error("fc_decode_tp: a stamped x needs 8-byte alignment");
        return Q4FC_EALIGN;
    }
    if (int rc = check_fc_args("fc_decode_tp", static_cast<const float*>(x), rows, K, ldx, wq, Ng, Kg, qtype, group_k,
                               N, reinterpret_cast<float*>(site->y_peer[0]), ldy))
        return rc;
    if (rows > kMaxDecodeRows) {
        set_error("fc_decode_tp: rows=%lld exceeds %d", (long long)rows, kMaxDecodeRows);
        return Q4FC_ELIMIT;
    }
    return launch_fc_decode_ring_tp(static_cast<const float*>(x), (int)rows, K, ldx,
                                       static_cast<const uint8_t*>(wq), Ng, Kg, qtype, group_k, N, ldy, flags,
                                       static_cast<cudaStream_t>(stream), site);
}

int q4fc_fc_decode_tp_batch(const q4fc_tp_call* calls, const q4fc_tp_site* const* sites, int ncalls, int qtype,
                            int group_k, unsigned flags, q4fc_stream_t stream) {
    if (!calls || !sites || ncalls < 1 || ncalls > 4) {
        set_error("fc_decode_tp_batch: null argument or ncalls=%d outside 1..4", ncalls);
        return Q4FC_EINVAL;
    }
    if (flags & Q4FC_FLAG_STREAMK) {
        set_error("fc_decode_tp_batch: Q4FC_FLAG_STREAMK is not available for the multi-GPU form");
        return Q4FC_EINVAL;
    }
    for (int i = 0; i < ncalls; i++) {
        const q4fc_tp_call& c = calls[i];
        const q4fc_tp_site* t = sites[i];
        if (!t || t->world < 1 || t->world > 8 || !t->epoch || !t->status || t->world != sites[0]->world ||
            t->epoch != sites[0]->epoch || t->status != sites[0]->status || t->x_stamped != sites[0]->x_stamped) {
            set_error("fc_decode_tp_batch: site %d is null, malformed, or differs from site 0 in world / epoch / status", i);
            return Q4FC_EINVAL;
        }
        if ((c.x == nullptr) == (c.xq == nullptr) || (c.x && c.x != calls[0].x) || (c.xq && t->x_stamped)) {
            set_error("fc_decode_tp_batch: call %d: exactly one of x (shared by all calls) and xq must be given", i);
            return Q4FC_EINVAL;
        }
        if (t->col_off < 0 || t->col_off % 32 != 0 || t->col_off + c.N > c.ldy) {
            set_error("fc_decode_tp_batch: call %d: col_off must be a multiple of 32 with col_off + N <= ldy", i);
            return Q4FC_EINVAL;
        }
        for (int r = 0; r < t->world; r++)
            if (!t->y_peer[r] || !aligned(t->y_peer[r], 8)) {
                set_error("fc_decode_tp_batch: call %d: y_peer[%d] is null or not 8-byte aligned", i, r);
                return Q4FC_EINVAL;
            }
        if (c.xq)
            if (int rc = check_xq_args("fc_decode_tp_batch", c.rows, c.K, group_k, c.xq)) return rc;
        if (c.x && t->x_stamped && !aligned(c.x, 8)) {
            set_error("fc_decode_tp_batch: a stamped x needs 8-byte alignment");
            return Q4FC_EALIGN;
        }
        if (int rc = check_fc_args("fc_decode_tp_batch", static_cast<const float*>(c.x ? c.x : c.xq), c.rows, c.K,
                                   c.x ? c.ldx : c.K, c.wq, c.Ng, c.Kg, qtype, group_k, c.N,
                                   reinterpret_cast<float*>(t->y_peer[0]), c.ldy))
            return rc;
        if (c.rows > kMaxDecodeRows) {
            set_error("fc_decode_tp_batch: rows=%lld exceeds %d", (long long)c.rows, kMaxDecodeRows);
            return Q4FC_ELIMIT;
        }
    }
    return launch_fc_decode_ring_tp_batch(calls, sites, ncalls, qtype, group_k, flags, static_cast<cudaStream_t>(stream));
}

int q4fc_tp_collect_multi(const unsigned long long* const* stamped, const int64_t* rows, const int64_t* N,
                          const int64_t* ld, float* const* dst, const int64_t* ldd, int n,
                          const unsigned long long* epoch, int* status, q4fc_stream_t stream) {
    if (!stamped || !rows || !N || !ld || !epoch || !status || n < 1 || n > 16) {
        set_error("tp_collect_multi: null argument or n=%d outside 1..16", n);
        return Q4FC_EINVAL;
    }
    for (int i = 0; i < n; i++)
        if (!stamped[i] || !aligned(stamped[i], 8) || rows[i] < 0 || N[i] < 0 || ld[i] < N[i] ||
            (dst && dst[i] && (!ldd || ldd[i] < N[i]))) {
            set_error("tp_collect_multi: buffer %d: null or misaligned pointer, negative size, or pitch smaller than N", i);
            return Q4FC_EINVAL;
        }
    return launch_tp_collect_multi(stamped, rows, N, ld, dst, ldd, n, epoch, status, static_cast<cudaStream_t>(stream));
}

int q4fc_fc_chain_create(const q4fc_chain_step* steps, int nsteps, const q4fc_fc_job* jobs, int njobs, int64_t rows,
                         int qtype, int group_k, void** chain) {
    if (!valid_variant(qtype, group_k)) {
        set_error("fc_chain: qtype=%d, group_k=%d is not a block type", qtype, group_k);
        return Q4FC_EVARIANT;
    }
    if (!steps || !jobs || !chain || nsteps <= 0 || njobs <= 0) {
        set_error("fc_chain: null pointer or no steps");
        return Q4FC_EINVAL;
    }
    if (rows < 1 || rows > kMaxDecodeRows) {
        set_error("fc_chain: rows=%lld outside 1..%d", (long long)rows, kMaxDecodeRows);
        return Q4FC_ELIMIT;
    }
    *chain = nullptr;
    return chain_create(steps, nsteps, jobs, njobs, (int)rows, qtype, group_k, chain);
}

int q4fc_fc_chain_run(void* chain, q4fc_stream_t stream) {
    if (!chain) {
        set_error("fc_chain: null handle");
        return Q4FC_EINVAL;
    }
    return chain_run(chain, static_cast<cudaStream_t>(stream));
}

int q4fc_fc_chain_check(void* chain, q4fc_stream_t stream) {
    if (!chain) {
        set_error("fc_chain: null handle");
        return Q4FC_EINVAL;
    }
    return chain_check(chain, static_cast<cudaStream_t>(stream));
}

int q4fc_fc_chain_destroy(void* chain) { return chain_destroy(chain); }

int q4fc_q8c_pack(const float* w, int64_t N, int64_t K, int8_t* wq, float* wscales, q4fc_stream_t stream) {
    if (N < 0 || K < 0) {
        set_error("q8c_pack: negative size");
        return Q4FC_EINVAL;
    }
    if (N == 0) return Q4FC_OK;
    if (!w || !wq || !wscales) {
        set_error("q8c_pack: null pointer");
        return Q4FC_EINVAL;
    }
    if (!aligned(wq, 4)) {
        set_error("q8c_pack: wq needs 4-byte alignment");
        return Q4FC_EALIGN;
    }
    return launch_q8c_pack(w, N, K, wq, wscales, static_cast<cudaStream_t>(stream));
}

size_t q4fc_q8c_workspace_bytes(int64_t rows, int64_t K) {
    if (rows < 0 || K < 0) return 0;
    return q8c_workspace_bytes(rows, K);
}

int q4fc_q8c_fc(const float* x, int64_t rows, int64_t K, int64_t ldx, const int8_t* wq, const float* wscales,
                int64_t Ng, int64_t Kg, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes,
                q4fc_stream_t stream) {
    if (rows < 0 || K < 0 || N < 0 || Ng < 0 || Kg < 0) {
        set_error("q8c_fc: negative size");
        return Q4FC_EINVAL;
    }
    if (Kg != (K + 31) / 32 || N > Ng * 32) {
        set_error("q8c_fc: weights [%lld][%lld][1024] do not match K=%lld, N=%lld", (long long)Ng, (long long)Kg,
                  (long long)K, (long long)N);
        return Q4FC_EINVAL;
    }
    if (rows == 0 || N == 0) return Q4FC_OK;
    if (!y || !wscales || (K > 0 && (!x || !wq))) {
        set_error("q8c_fc: null pointer");
        return Q4FC_EINVAL;
    }
    if (ldx < K || ldy < N) {
        set_error("q8c_fc: ldx=%lld / ldy=%lld smaller than K=%lld / N=%lld", (long long)ldx, (long long)ldy,
                  (long long)K, (long long)N);
        return Q4FC_EINVAL;
    }
    if (!aligned(wq, 16) || !aligned(x, 4)) {
        set_error("q8c_fc: wq needs 16-byte and x 4-byte alignment");
        return Q4FC_EALIGN;
    }
    if (K > 0 && (!ws || ws_bytes < q8c_workspace_bytes(rows, K))) {
        set_error("q8c_fc: workspace of %zu bytes, need %zu", ws ? ws_bytes : (size_t)0, q8c_workspace_bytes(rows, K));
        return Q4FC_EWORKSPACE;
    }
    if (ws && !aligned(ws, 256)) {
        set_error("q8c_fc: workspace needs 256-byte alignment");
        return Q4FC_EALIGN;
    }
    return launch_q8c_fc(x, rows, K, ldx, wq, wscales, Ng, Kg, N, y, ldy, ws, static_cast<cudaStream_t>(stream));
}

int q4fc_emb_q8c_quant(const float* table, int64_t V, int64_t E, int8_t* codes, float* scales, q4fc_stream_t stream) {
    if (V < 0 || E < 0) {
        set_error("emb_q8c_quant: negative size");
        return Q4FC_EINVAL;
    }
    if (V == 0) return Q4FC_OK;
    if (!scales || (E > 0 && (!table || !codes))) {
        set_error("emb_q8c_quant: null pointer");
        return Q4FC_EINVAL;
    }
    return launch_emb_q8c_quant(table, V, E, codes, scales, static_cast<cudaStream_t>(stream));
}

int q4fc_emb_q8c(const void* ids, int ids_are_i32, int64_t n, const int8_t* codes, const float* scales, int64_t V,
                 int64_t E, float* out, int64_t ldo, q4fc_stream_t stream) {
    if (n < 0 || V < 0 || E < 0) {
        set_error("emb_q8c: negative size");
        return Q4FC_EINVAL;
    }
    if (n == 0 || E == 0) return Q4FC_OK;
    if (!ids || !codes || !scales || !out) {
        set_error("emb_q8c: null pointer");
        return Q4FC_EINVAL;
    }
    if (ldo < E) {
        set_error("emb_q8c: ldo=%lld smaller than E=%lld", (long long)ldo, (long long)E);
        return Q4FC_EINVAL;
    }
    return launch_emb_q8c(ids, ids_are_i32, n, codes, scales, V, E, out, ldo, static_cast<cudaStream_t>(stream));
}

int q4fc_fc_check_status(void* ws, q4fc_stream_t stream) {
    if (!ws) {
        ws = ring_status_word();
        if (!ws) return Q4FC_ECUDA;
    }
    int status = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    Q4FC_CUDA_OK(cudaMemcpyAsync(&status, ws, sizeof(int), cudaMemcpyDeviceToHost, s));
    Q4FC_CUDA_OK(cudaStreamSynchronize(s));
    if (status != 0) {
        Q4FC_CUDA_OK(cudaMemsetAsync(ws, 0, sizeof(int), s));
        set_error("device status word = 0x%x (%s)", status,
                  (status & 0x100) ? "an embedding id was out of range" : "a bounded wait ran out");
        return Q4FC_EDEVICE;
    }
    return Q4FC_OK;
}

}  // extern "C"
