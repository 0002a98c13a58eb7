// Prefill FC (rows > 8).  Interim form: the rows are walked eight at a time
// through the decode kernel, so the packed weights are re-read rows/8 times
// (from L2 when they fit).  Replaces fc_Q4A (ops/op_fc.hpp:286-426) for large
// B*M with the same arithmetic as the decode path.
#include "common.cuh"

namespace q4fc {

size_t prefill_workspace_bytes(int64_t rows, int64_t K, int64_t N, int qtype, int G) {
    (void)rows, (void)K, (void)qtype, (void)G;
    return decode_workspace_bytes(N);
}

int launch_fc_prefill(const float* x, int64_t rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng,
                      int64_t Kg, int qtype, int G, int64_t N, float* y, int64_t ldy, void* ws, size_t ws_bytes,
                      unsigned flags, cudaStream_t s) {
    for (int64_t r = 0; r < rows; r += kMaxDecodeRows) {
        const int n = (int)((rows - r < kMaxDecodeRows) ? rows - r : kMaxDecodeRows);
        (void)ws, (void)ws_bytes;
        int rc = launch_fc_decode_cluster(x + r * ldx, n, K, ldx, wq, Ng, Kg, qtype, G, N, y + r * ldy, ldy,
                                          flags & ~Q4FC_FLAG_PDL, s);
        if (rc) return rc;
    }
    return Q4FC_OK;
}

}  // namespace q4fc
