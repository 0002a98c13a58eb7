/*
 * q4fc_b200 -- C-ABI of the B200 (sm_100a) quantized fully-connected path.
 *
 * Drop-in boundary for the Q4_0 / Q4_1 FC of usstq/llama.cl: the entry points
 * below are what a binding of that project's FC ops would call instead of its
 * CPU code.  Plain pointers and sizes only; every pointer is a DEVICE pointer
 * unless stated otherwise; every call is asynchronous on `stream` and
 * allocates nothing (the two exceptions, q4fc_tp_arena_create / _open, say
 * so).  All functions return 0 on success or a Q4FC_E* code and
 * never throw or abort; q4fc_last_error() gives the detail text of the last
 * failure on the calling thread.
 *
 * Packed weight tensor (identical, byte for byte, to the reference's):
 *   int8 [Ng][Kg][BS],  Ng = ceil(N/32), Kg = ceil(K/G), one block = 32
 *   columns x G k:  G/8 rows of 128 bytes (byte n*4 + (k&3) of row k>>3 holds
 *   k in its low nibble when ((k>>2)&1)==0, else in its high nibble), then
 *   32 fp16 scales, then (Q4_1 only) 32 fp16 minima.
 *   BS = 16*G + 64 (Q4_0) or 16*G + 128 (Q4_1): 576 / 2112 / 640 / 2176.
 *   (reference: ops/op_fc.hpp:14-24, 39-48, 64-71)
 */
#ifndef Q4FC_B200_H
#define Q4FC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with hidden visibility */
#endif

/* cudaStream_t, passed as an opaque pointer so that this header needs no CUDA include */
typedef void* q4fc_stream_t;

enum {
    Q4FC_Q4_0 = 0, /* symmetric, levels -7..7, no minimum   (ops/op_fc.hpp:64)  */
    Q4FC_Q4_1 = 1  /* asymmetric, levels 0..15 + minimum    (ops/op_fc.hpp:14)  */
};

enum {
    Q4FC_OK = 0,
    Q4FC_EINVAL = 1,    /* bad size, null pointer, N not covered by Ng, K not covered by Kg */
    Q4FC_EVARIANT = 2,  /* (qtype, group_k) is not one of the four block types */
    Q4FC_EALIGN = 3,    /* a pointer or leading dimension misses its alignment */
    Q4FC_EWORKSPACE = 4,/* workspace missing or smaller than q4fc_fc_workspace_bytes() */
    Q4FC_ECUDA = 5,     /* a CUDA runtime call failed (launch, attribute) */
    Q4FC_EDEVICE = 6,   /* a kernel reported a bounded wait that ran out */
    Q4FC_ELIMIT = 7     /* size beyond a stated maximum of the entry point */
};

/* flags of q4fc_fc* */
enum {
    /* Q4_0 only: sign-extend the stored nibble.  Off by default because the
     * reference reads it unsigned (ops/op_fc.hpp:95-106, 364-376) and parity
     * is defined against that. */
    Q4FC_FLAG_NIBBLE_SIGNED = 1u,
    /* Launch with programmatic stream serialization: the kernel may start
     * while its predecessor on the stream drains; it touches activations,
     * outputs and workspace only after the predecessor has completed, and
     * streams weights before that.  Use only when the predecessor does not
     * write this call's weights. */
    Q4FC_FLAG_PDL = 2u,
    /* q4fc_fc_decode only: use the stream-K kernel (one contiguous byte run
     * per CTA, weights staged in registers, partial sums through the workspace)
     * instead of the default kernel (weights staged in a shared-memory ring by
     * bulk copies, partial sums through shared memory, no workspace needed).
     * Same results within rounding of the fp32 sums. */
    Q4FC_FLAG_STREAMK = 4u,
    /* q4fc_fc_decode with a workspace: always quantize the activations in a small launch of their own in
     * front of the FC kernel (by default only for large rows x K).  The FC kernel otherwise quantizes
     * them itself, every CTA its own copy: the shortest path for one call at a time, but repeated work.
     * Codes, scales and outputs are the same bit for bit. */
    Q4FC_FLAG_PREQUANT = 8u
};

int q4fc_version(void);
const char* q4fc_strerror(int code);
const char* q4fc_last_error(void);

/* Block size in bytes, or -1 for an unknown variant.  (sizeof(q4_block), ops/op_fc.hpp:109) */
int q4fc_block_bytes(int qtype, int group_k);
/* Recover (qtype, group_k) from the last dimension of a packed tensor. */
int q4fc_infer_variant(int block_bytes, int* qtype, int* group_k);

/* Replaces offline_FC_quant_Q4A (ops/op_fc.hpp:151-219; old extension
 * FC_quant_Q4A, ext/llama_ext.cpp:405-471).
 * w: fp32 [N][K] row-major (16-byte aligned, K % 4 == 0).  wq: [Ng][Kg][BS].
 * Bit-exact with the reference for K % group_k == 0.  Columns n >= N get zero
 * scale, minimum and nibbles (the reference leaves those nibbles
 * uninitialised); a ragged last K group is scanned over its valid part only. */
int q4fc_pack(const float* w, int64_t N, int64_t K, int qtype, int group_k, void* wq, q4fc_stream_t stream);

/* Replaces offline_FC_dequant_Q4A (ops/op_fc.hpp:124-149).
 * out: fp32 [Ng*32][Kg*group_k].  nibble_signed = 0 reproduces the reference
 * (unsigned nibble for both block types). */
int q4fc_dequant(const void* wq, int64_t Ng, int64_t Kg, int qtype, int group_k, int nibble_signed, float* out,
                 q4fc_stream_t stream);

/* Replaces FC_dynamic_quantize_x (ops/op_fc.hpp:221-272, with get_amax and
 * quant_row_q8_0 of ops/utils.hpp:177-220).  x: fp32 [rows][K] with row
 * stride ldx.  codes: int8 [rows][Kg*group_k]; scales, gsums: fp32
 * [rows][Kg] (gsums may be NULL).  scale = 1 for Q4_1, 1/16 for Q4_0 as in
 * ops/op_fc.hpp:315.  Codes, scales and group sums are bit-exact (the sums
 * are accumulated sequentially like the reference's). */
int q4fc_quant_x(const float* x, int64_t rows, int64_t K, int64_t ldx, int group_k, float scale, int8_t* codes,
                 float* scales, float* gsums, q4fc_stream_t stream);

/* Replaces fc_Q4A (ops/op_fc.hpp:286-426; old extension FC_evaluate_Q4A,
 * ext/llama_ext.cpp:484-606): y[r][n] = quantized(x[r]) . W[n], r < rows,
 * n < N.  x: fp32 [rows][K] (row stride ldx), y: fp32 [rows][N] (row stride
 * ldy).  rows is the reference's B*M.  The activation quantization happens
 * inside, as in the reference.
 *   q4fc_fc_decode  rows <= 8: weight-streaming GEMV, HBM-bound.
 *   q4fc_fc_prefill any rows:  int8 tensor-core GEMM.
 *   q4fc_fc         picks one of the two.
 * ws: workspace of at least q4fc_fc_workspace_bytes() bytes, 256-byte
 * aligned, zeroed once with q4fc_fc_workspace_init() before its first use;
 * the kernels leave it ready for the next call.  Calls that may overlap on
 * the GPU need separate workspaces.  q4fc_fc_decode without
 * Q4FC_FLAG_STREAMK accepts ws = NULL; given a workspace it uses it, when
 * rows x K is large (from about 40 thousand values), to quantize the
 * activations once in a small launch of its own in front of the FC kernel
 * instead of inside it -- same results bit for bit, less repeated work.
 * With Q4FC_FLAG_STREAMK, N <= 524288. */
size_t q4fc_fc_workspace_bytes(int64_t rows, int64_t K, int64_t N, int qtype, int group_k);
int q4fc_fc_workspace_init(void* ws, size_t ws_bytes, q4fc_stream_t stream);
int q4fc_fc_decode(const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg,
                   int qtype, int group_k, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes,
                   unsigned flags, q4fc_stream_t stream);
int q4fc_fc_prefill(const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg,
                    int qtype, int group_k, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes,
                    unsigned flags, q4fc_stream_t stream);
int q4fc_fc(const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg, int qtype,
            int group_k, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes, unsigned flags,
            q4fc_stream_t stream);

/* q4fc_fc_decode with the addition that follows the FC in the reference folded into the kernel's last step:
 * y = fc(x) + addend, one fp32 add per output as llmops.iadd does (ops/op_misc.hpp:55-79) -- the bias
 * (chatllama/main.py:166-167; ld_addend = 0: addend is one row of N values used for every row) or the residual
 * stream (chatllama/main.py:356, 372; addend is [rows][ld_addend] and may be y itself).  rows <= 8; the
 * stream-K flag is not accepted. */
int q4fc_fc_decode_add(const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg,
                       int qtype, int group_k, int64_t N, float* y, int64_t ldy, const float* addend,
                       int64_t ld_addend, void* ws, size_t ws_bytes, unsigned flags, q4fc_stream_t stream);

/* Several FCs that read the same input, as one launch: the q, k and v projections of an attention block
 * (chatllama/main.py:348-350), or gate and up of the MLP (chatllama/main.py:365-367) -- in the reference three
 * and two calls of fc_Q4A on one tensor.  Every job is one packed weight tensor of the same block type and the
 * same Kg with its own output (and optional addend, as q4fc_fc_decode_add); the stripes of all jobs are dealt
 * over the SMs as one list, so short outputs share a launch instead of each paying its own start and end.
 * njobs 1..4, rows <= 8.  x: fp32 [rows][ldx], or NULL with xq != NULL: a buffer made by q4fc_quant_x_q8 /
 * q4fc_rmsnorm_quant / q4fc_silu_mul_quant (then ldx is ignored).  Each output equals what q4fc_fc_decode /
 * q4fc_fc_decode_q8 gives for that job alone, within the rounding of the fp32 sums (the jobs' stripes are
 * cut over the SMs differently than a single call's). */
typedef struct q4fc_fc_job {
    const void* wq;      /* packed [Ng][Kg][BS] */
    int64_t Ng;
    int64_t N;           /* N <= 32 * Ng */
    float* y;            /* fp32 [rows][ldy] */
    int64_t ldy;
    const float* addend; /* NULL, or as in q4fc_fc_decode_add */
    int64_t ld_addend;
} q4fc_fc_job;
int q4fc_fc_decode_multi(const float* x, const void* xq, int64_t rows, int64_t K, int64_t ldx, int64_t Kg, int qtype,
                         int group_k, const q4fc_fc_job* jobs, int njobs, void* ws, size_t ws_bytes, unsigned flags,
                         q4fc_stream_t stream);

/* A batch of independent FCs as ONE launch: up to 16 calls of one block type, each with its own weights, output
 * and pre-quantized input (calls may share an input: pass the same xq pointer).  The reference runs such calls
 * one after the other (every fc_Q4A of ops/perf_ops.py:239-242, or of a model step, is a call of its own); here
 * the stripes of all calls are dealt over the SMs as one list of about equal bytes per SM, so the whole batch
 * streams without a kernel boundary in it -- on B200 a single 9 MB FC is over in the time a launch takes to
 * start and end, while sixteen of them in one launch run at the pace of the memory system.  Every output is
 * what q4fc_fc_decode_q8 gives for that call alone, within the rounding of the fp32 sums.  rows <= 8. */
typedef struct q4fc_fc_call {
    const void* xq;      /* q4fc_xq_bytes(rows, K, group_k) bytes made by q4fc_quant_x_q8 / q4fc_rmsnorm_quant / ... */
    int64_t rows, K;
    const void* wq;      /* packed [Ng][Kg][BS] */
    int64_t Ng, Kg, N;
    float* y;            /* fp32 [rows][ldy] */
    int64_t ldy;
    const float* addend; /* NULL, or as in q4fc_fc_decode_add */
    int64_t ld_addend;
} q4fc_fc_call;
int q4fc_fc_decode_batch(const q4fc_fc_call* calls, int ncalls, int qtype, int group_k, unsigned flags,
                         q4fc_stream_t stream);

/* ---- activations quantized once, used by several FCs ------------------------------------------------
 * In the reference every FC quantizes its input itself, so the output of one normalization is quantized
 * three times (q, k, v projections) or twice (gate, up) -- chatllama/main.py:344-368.  These entry points
 * split the two steps.  xq is a device buffer of q4fc_xq_bytes(rows, K, group_k) bytes, 256-byte aligned:
 * int8 codes [rows][Kg*group_k], then (256-byte aligned) fp32 [Kg][16] with entry 2m = scale of row m and
 * entry 2m+1 = group sum of row m (Q4_1), or the bits of 8 * sum of codes with want_isum (Q4_0 with
 * Q4FC_FLAG_NIBBLE_SIGNED).  rows <= 8.  Codes and scales are bit-equal to FC_dynamic_quantize_x
 * (ops/op_fc.hpp:221-272); q4fc_fc_decode_q8 on them gives the bytes q4fc_fc_decode gives on the fp32 input.
 *   q4fc_quant_x_q8      the quantizer alone.
 *   q4fc_rmsnorm_quant   replaces llmops.rmsnorm (ops/op_misc.hpp:142-181) + that quantizer: normalizes each
 *                        row (bit-equal to the reference: same eight running sums, same fold, IEEE division
 *                        and square root) and quantizes it; y (fp32 [rows][ldy]) receives the normalized
 *                        values unless NULL.  K % 8 == 0 as in the reference, x / weight / y 16-byte aligned.
 *   q4fc_add_rmsnorm_quant  the same with the residual addition in front of it (llmops.iadd,
 *                        chatllama/main.py:359): the row that is normalized is x + residual, and sum_out
 *                        (may be NULL, may alias x or residual) receives that sum -- the new residual
 *                        stream.  residual and sum_out share x's row stride ldx.
 *   q4fc_silu_mul_quant  replaces llmops.itrans(gate, "silu") + llmops.imul(up, gate) (ops/op_misc.hpp:83-138,
 *                        chatllama/main.py:365-368) + that quantizer: the value quantized is silu(gate) * up, the
 *                        input of the down projection; prod (fp32 [rows][ldp], may be NULL) receives it.  gate and
 *                        up share the row stride ld.  The reference evaluates the sigmoid with a polynomial exp
 *                        and _mm256_rcp_ps (relative error up to 3.7e-4); here it is expf and an IEEE division, so
 *                        the products agree to about 4e-4 relative -- inside the 1e-3 / 1e-4 tolerance of fp32
 *                        outputs, not bit for bit -- and the codes are exact given those products.
 *   q4fc_fc_decode_q8    the decode FC on such a buffer. */
size_t q4fc_xq_bytes(int64_t rows, int64_t K, int group_k);
int q4fc_quant_x_q8(const float* x, int64_t rows, int64_t K, int64_t ldx, int group_k, int want_isum, void* xq,
                    unsigned flags, q4fc_stream_t stream);
/* q4fc_quant_x_q8 for up to 16 inputs in ONE launch (the inputs of a batch of independent FCs): the same codes,
 * scales and sums as one call per input.  All inputs share group_k and want_isum. */
typedef struct q4fc_xq_call {
    const float* x; /* fp32 [rows][ldx] */
    int64_t rows;   /* <= 8 */
    int64_t K;
    int64_t ldx;
    void* xq;       /* q4fc_xq_bytes(rows, K, group_k) bytes, 256-byte aligned */
} q4fc_xq_call;
int q4fc_quant_x_q8_batch(const q4fc_xq_call* calls, int ncalls, int group_k, int want_isum, unsigned flags,
                          q4fc_stream_t stream);
int q4fc_rmsnorm_quant(const float* x, int64_t rows, int64_t K, int64_t ldx, const float* weight, float eps, float* y,
                       int64_t ldy, int group_k, int want_isum, void* xq, unsigned flags, q4fc_stream_t stream);
int q4fc_add_rmsnorm_quant(const float* x, const float* residual, float* sum_out, int64_t rows, int64_t K, int64_t ldx,
                           const float* weight, float eps, float* y, int64_t ldy, int group_k, int want_isum,
                           void* xq, unsigned flags, q4fc_stream_t stream);
int q4fc_silu_mul_quant(const float* gate, const float* up, int64_t rows, int64_t K, int64_t ld, float* prod, int64_t ldp,
                        int group_k, int want_isum, void* xq, unsigned flags, q4fc_stream_t stream);
int q4fc_fc_decode_q8(const void* xq, int64_t rows, int64_t K, const void* wq, int64_t Ng, int64_t Kg, int qtype,
                      int group_k, int64_t N, float* y, int64_t ldy, unsigned flags, q4fc_stream_t stream);

/* No counterpart in the reference.  q4fc_fc_decode for callers that cannot
 * allocate device memory -- hosts that give all of it to their own arena at
 * start-up, or that run under a budget where a late cudaMalloc may fail or
 * stall the device.  The reduction scratch is a fixed array inside the
 * library image (about 1.3 MB per GPU that loads the library, held until the
 * process exits), so no workspace is passed and nothing is allocated.
 * Limits: rows <= 8, N <= 262144, at most 320 SMs; beyond them the call
 * returns Q4FC_ELIMIT.  All calls on a device share the array: calls that may
 * overlap on the GPU race, so keep them ordered on one stream (or by events).
 * The first call on a device looks up the array's address; make it outside
 * any stream capture.  Results are identical to q4fc_fc_decode. */
int q4fc_fc_decode_noalloc(const float* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng,
                           int64_t Kg, int qtype, int group_k, int64_t N, float* y, int64_t ldy, unsigned flags,
                           q4fc_stream_t stream);

/* ---- one FC split along N over the GPUs of a node, joined inside the kernel ----
 * No counterpart in the reference (it has no multi-device code).  Each rank
 * holds the contiguous stripe range [nb0, nb1) of the packed tensor.  Outputs
 * travel as 8-byte "stamped" words: the fp32 value in the low half, the low 32
 * bits of a step counter (the "epoch") in the high half.  The decode kernel
 * stores its columns, stamped, straight into the output buffer of EVERY rank
 * (peer-mapped pointers, plain 64-bit stores over NVLink).  A 64-bit store is
 * indivisible, so a reader that finds the current epoch in a word has its value
 * too: no fence, no flag, no collective call, no extra launch.  An FC whose
 * input is such a buffer (x_stamped) re-reads each word until its stamp is the
 * current epoch (bounded: after one second *status becomes non-zero and the
 * kernel carries on; once it is non-zero later waits end at once).
 *
 * The shared memory comes from an "arena": cudaMalloc'ed and zeroed by
 * q4fc_tp_arena_create, exported as a 64-byte CUDA IPC handle that the host
 * ships to the other ranks by any transport, and mapped there with
 * q4fc_tp_arena_open (peer access over NVLink).  Every rank lays its arena out
 * identically, so a peer's pointer is its mapped base plus the local offset.
 *
 * An epoch belongs to a "schedule": a fixed set of FC calls that run together,
 * each exactly once per step.  Per step each rank calls q4fc_tp_step_begin once
 * before the schedule's first FC: it adds 1 to the local epoch and is a barrier
 * over the ranks (bounded the same way), so nobody overwrites a buffer that a
 * slower rank is still reading from the step before.  Independent work gets
 * its own epoch and barrier words.  q4fc_tp_collect unpacks a stamped buffer
 * into plain floats, waiting for every word -- the hand-over to consumers that
 * are not FC kernels.  All of it can be captured in a CUDA graph: the epoch
 * lives in device memory. */
typedef struct q4fc_tp_site {
    int world;                       /* ranks, 1..8 */
    int x_stamped;                   /* x is a stamped buffer of this rank (ldx counts 8-byte words) */
    int64_t col_off;                 /* first output column of this rank's slice: 32 * nb0 */
    unsigned long long* y_peer[8];   /* every rank's stamped output [rows, ldy], own rank included */
    const unsigned long long* epoch; /* local step counter, advanced by q4fc_tp_step_begin */
    int* status;                     /* local int, set non-zero when a bounded wait ran out */
    void* xq_scratch;                /* NULL, or q4fc_xq_bytes(rows, K, group_k) bytes of local scratch (256-byte
                                        aligned): with a plain fp32 x the activations are then quantized once in a
                                        small launch in front of the FC kernel (as Q4FC_FLAG_PREQUANT does for
                                        q4fc_fc_decode) instead of by every cluster; ignored with x_stamped */
} q4fc_tp_site;

/* sizeof(q4fc_tp_site) as the library was built: bindings that mirror the struct check theirs against it */
size_t q4fc_tp_site_bytes(void);
int q4fc_tp_arena_create(size_t bytes, void** base, void* ipc_handle_64);
int q4fc_tp_arena_open(const void* ipc_handle_64, void** peer_base);
int q4fc_tp_arena_close(void* peer_base);
int q4fc_tp_arena_destroy(void* base);
/* barrier_peer[r]: rank r's barrier counter (own rank included), barrier_local: this rank's. */
int q4fc_tp_step_begin(unsigned long long* epoch, unsigned long long* const* barrier_peer,
                       const unsigned long long* barrier_local, int world, int* status, q4fc_stream_t stream);
/* stamped [rows, ld] (this rank's buffer) -> dst fp32 [rows, ldd], columns [0, N). */
int q4fc_tp_collect(const unsigned long long* stamped, int64_t rows, int64_t N, int64_t ld, float* dst, int64_t ldd,
                    const unsigned long long* epoch, int* status, q4fc_stream_t stream);
/* x: fp32 [rows, ldx], or with site->x_stamped a stamped buffer passed through the same pointer.
 * N, Ng: this rank's slice (N = 32 * Ng except on the rank holding the ragged tail); ldy: row pitch of the
 * stamped output in words.  rows <= 8.  flags as q4fc_fc_decode (Q4FC_FLAG_STREAMK is not accepted). */
int q4fc_fc_decode_tp(const void* x, int64_t rows, int64_t K, int64_t ldx, const void* wq, int64_t Ng, int64_t Kg,
                      int qtype, int group_k, int64_t N, int64_t ldy, const q4fc_tp_site* site, unsigned flags,
                      q4fc_stream_t stream);

/* Up to four N-split FCs as ONE launch (q/k/v, gate/up, or four independent calls of a batch).  Call i stores
 * into sites[i]->y_peer at sites[i]->col_off; world, epoch, status and x_stamped are taken from sites[0] and
 * must be the same in all.  Inputs: every call its own pre-quantized xq (x = NULL), or all calls the same x
 * (fp32 [rows][ldx], or a stamped buffer with sites[0]->x_stamped), quantized inside the kernel. */
typedef struct q4fc_tp_call {
    const void* x;   /* fp32 / stamped input shared by all calls, or NULL */
    const void* xq;  /* pre-quantized input of this call, or NULL */
    int64_t rows, K, ldx;
    const void* wq;  /* this rank's stripes [Ng][Kg][BS] */
    int64_t Ng, Kg, N, ldy;
} q4fc_tp_call;
int q4fc_fc_decode_tp_batch(const q4fc_tp_call* calls, const q4fc_tp_site* const* sites, int ncalls, int qtype,
                            int group_k, unsigned flags, q4fc_stream_t stream);
/* q4fc_tp_collect for up to 16 stamped buffers in one launch.  dst[i] may be NULL: then the launch only waits until
 * every word of buffer i carries the current epoch (the step's hand-over to consumers that read stamped words). */
int q4fc_tp_collect_multi(const unsigned long long* const* stamped, const int64_t* rows, const int64_t* N,
                          const int64_t* ld, float* const* dst, const int64_t* ldd, int n,
                          const unsigned long long* epoch, int* status, q4fc_stream_t stream);

/* ---- a chain of dependent decode FCs in one launch -------------------------------------------------------------
 *
 * Replaces a run of the reference's Model.forward (chatllama/main.py:331-380): per layer the fc_Q4A calls q, k, v |
 * o | gate, up | down, each fed by the one before through llmops.rmsnorm (ops/op_misc.hpp:142-181), llmops.iadd
 * (:55-79), llmops.itrans("silu") and llmops.imul (:83-138), and lm_head at the end.  One persistent kernel runs all
 * steps: the weight stream never stops at a step boundary, only the activations wait (a grid barrier per step).
 *
 * A step: one input x (fp32 [rows][ldx], rows <= 8, K % 8 == 0, 16-byte aligned, ldx % 4 == 0; written by an earlier
 * step of the chain or by work ordered before the launch), a transform applied to it before it is quantized
 *   Q4FC_CHAIN_PLAIN     none
 *   Q4FC_CHAIN_RMSNORM   (x / sqrt(mean(x^2) + eps)) * aux[k]          aux: fp32 [K]
 *   Q4FC_CHAIN_SILU_MUL  aux[m][k] * silu(x[m][k])                     aux: fp32 [rows][ldx] (the up projection)
 * and njobs >= 1 jobs (q4fc_fc_job: weights, output, optional addend = bias or residual) that multiply it; the jobs
 * of all steps follow one another in `jobs`.  A job must not write the input of its own step; a buffer may be
 * reused by later steps.  Per step the values are those of q4fc_rmsnorm_quant / q4fc_silu_mul_quant /
 * q4fc_quant_x_q8 followed by q4fc_fc_decode_multi (same codes bit for bit; outputs within rounding of the fp32 sums).
 *
 *   q4fc_fc_chain_create   checks the steps, uploads their tables (cudaMalloc + synchronous copies: not inside a
 *                          stream capture) and returns a handle bound to the current device.  The quantized input
 *                          of a step (rows x largest K bytes), the partial sums and the step tables share an SM's
 *                          shared memory with the weight ring: Q4FC_ELIMIT when less than two ring slots would be
 *                          left (a 32-layer Llama-7B chain fits with up to 4 rows), or when the tables exceed 40 KB.
 *   q4fc_fc_chain_run      one cooperative launch of one CTA per SM on `stream`; asynchronous; may be captured into
 *                          a CUDA graph.  Launches of one handle must not overlap on the GPU.
 *   q4fc_fc_chain_check    host-synchronous: Q4FC_OK, or Q4FC_EDEVICE when a bounded wait inside a launch ran out
 *                          (results invalid; the handle is usable again).
 *   q4fc_fc_chain_destroy  frees the handle (after its launches have completed). */
enum { Q4FC_CHAIN_PLAIN = 0, Q4FC_CHAIN_RMSNORM = 1, Q4FC_CHAIN_SILU_MUL = 2 };
typedef struct q4fc_chain_step {
    const float* x;
    int64_t ldx;
    int64_t K;
    int transform;
    float eps;        /* RMSNORM */
    const float* aux; /* RMSNORM: weight; SILU_MUL: up */
    int njobs;
} q4fc_chain_step;
int q4fc_fc_chain_create(const q4fc_chain_step* steps, int nsteps, const q4fc_fc_job* jobs, int njobs, int64_t rows,
                         int qtype, int group_k, void** chain);
int q4fc_fc_chain_run(void* chain, q4fc_stream_t stream);
int q4fc_fc_chain_check(void* chain, q4fc_stream_t stream);
int q4fc_fc_chain_destroy(void* chain);

/* ---- per-channel int8 weights ("Q8C"): the FC of the reference's older extension and its embedding table ------
 *
 *   q4fc_q8c_pack         replaces FC_quant_Q8C (ext/llama_ext.cpp:56-113).  w: fp32 row-major [N][K] on the device.
 *                         wq: int8 [Ng][Kg][1024] (Ng = ceil(N/32), Kg = ceil(K/32); q8_c_block,
 *                         ext/llama_ext.cpp:50-54), wscales: fp32 [Ng*32].  Bit-identical to the reference.
 *   q4fc_q8c_workspace_bytes / q4fc_q8c_fc
 *                         replace FC_evaluate_Q8C (ext/llama_ext.cpp:232-371): the activations are quantized per
 *                         32-group with scale 1 and no group sums (its FC_dynamic_quantize_x call, :360) into the
 *                         workspace, then y[m][n] = wscales[n] * sum over groups of dx[m][kb] * (codes . q).  The
 *                         integer sums are exact; the fp32 sum over groups is split over warps (and CTAs of a
 *                         cluster), so y agrees with the reference within fp32 rounding (1e-3 relative / 1e-4
 *                         absolute is the tested bound), the same from run to run.  Any rows >= 0; N need not be a
 *                         multiple of 32 (the reference stores whole 32-column groups and overruns its output
 *                         there).  ws: device scratch of q4fc_q8c_workspace_bytes(rows, K) bytes, 256-byte aligned.
 *   q4fc_emb_q8c_quant    replaces embedding_q8c_quant_w (ops/op_embedding.hpp:51-78): per row of the fp32 table
 *                         [V][E] one scale amax/127 and int8 codes [V][E].  Bit-identical to the reference.
 *   q4fc_emb_q8c          replaces embedding_q8c (ops/op_embedding.hpp:80-137): out[i][:] = scales[id] * codes[id][:]
 *                         for n ids (int64, or int32 when ids_are_i32 != 0) on the device; out fp32 [n][ldo].
 *                         Bit-identical.  The reference does not check the ids; here an id outside [0, V) gives a
 *                         row of zeros and sets the device status word that q4fc_fc_check_status(NULL, ..) reads. */
int q4fc_q8c_pack(const float* w, int64_t N, int64_t K, int8_t* wq, float* wscales, q4fc_stream_t stream);
size_t q4fc_q8c_workspace_bytes(int64_t rows, int64_t K);
int q4fc_q8c_fc(const float* x, int64_t rows, int64_t K, int64_t ldx, const int8_t* wq, const float* wscales,
                int64_t Ng, int64_t Kg, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes,
                q4fc_stream_t stream);
int q4fc_emb_q8c_quant(const float* table, int64_t V, int64_t E, int8_t* codes, float* scales, q4fc_stream_t stream);
int q4fc_emb_q8c(const void* ids, int ids_are_i32, int64_t n, const int8_t* codes, const float* scales, int64_t V,
                 int64_t E, float* out, int64_t ldo, q4fc_stream_t stream);

/* Reads and clears the device status word kept at the start of a workspace
 * (host-synchronous: waits for `stream`).  ws = NULL reads the word that decode
 * calls made without a workspace share (one per device).  Returns Q4FC_OK or
 * Q4FC_EDEVICE (a bounded wait inside a kernel ran out, or an embedding id was out of range; the results
 * are invalid). */
int q4fc_fc_check_status(void* ws, q4fc_stream_t stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* Q4FC_B200_H */
