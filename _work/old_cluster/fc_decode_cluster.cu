// Single-GPU instantiations of the cluster decode kernel (fc_decode_cluster_impl.cuh, TP = false).
#define Q4FC_TIMELINE_SETTER q4fc_debug_set_timeline
#include <cstdlib>

#include "fc_decode_cluster_impl.cuh"

namespace q4fc {

// Picks the number of clusters for a shape.  Every cluster quantizes the whole
// activation once (spread over its CTAs), so few large clusters are preferred.
// nc_cap is how many clusters may be resident at once; among the counts in
// (nc_cap/2, nc_cap] the one with the most even stripe split wins, and at most
// kMaxStripes stripes go to one cluster (more clusters than nc_cap, i.e. more
// than one wave, only for very large N).
int choose_cluster_count(int64_t Ng, int64_t nc_cap) {
    int64_t nc_hi = nc_cap < Ng ? nc_cap : Ng;
    if (nc_hi < 1) nc_hi = 1;
    const int64_t nc_lo = (Ng + kMaxStripes - 1) / kMaxStripes;
    if (nc_lo > nc_hi) return (int)nc_lo;
    int64_t best = nc_hi, best_r = (Ng + nc_hi - 1) / nc_hi;
    for (int64_t nc = nc_hi; nc >= nc_lo && nc > nc_hi / 2; nc--) {
        const int64_t r = (Ng + nc - 1) / nc;  // stripes of the busiest cluster
        if (r < best_r) best_r = r, best = nc;
    }
    // the smallest count that keeps the busiest cluster at best_r stripes wastes the fewest CTAs
    while (best - 1 >= nc_lo && (Ng + best - 2) / (best - 1) == best_r) best--;
    return (int)best;
}

int64_t pre_quant_min_values() {
    static const int64_t v = [] {
        const char* e = getenv("Q4FC_PREQUANT_MIN_VALUES");  // tuning aid: 0 = always, a huge value = never
        if (e && *e) return (int64_t)atoll(e);
        return kPreQuantMinValues;
    }();
    return v;
}

int launch_fc_decode_cluster(const float* x, int rows, int64_t K, int64_t ldx, const uint8_t* wq, int64_t Ng,
                             int64_t Kg, int qtype, int G, int64_t N, float* y, int64_t ldy, unsigned flags,
                             cudaStream_t s, void* ws, size_t ws_bytes, const void* xq, const float* addend,
                             int64_t addend_ld) {
    return launch_cluster_impl<false>(x, rows, K, ldx, wq, Ng, Kg, qtype, G, N, y, ldy, flags, s, nullptr, ws,
                                      ws_bytes, xq, addend, addend_ld);
}

}  // namespace q4fc
