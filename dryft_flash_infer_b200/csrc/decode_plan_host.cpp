// The decode attention's plan worked out on the host, by the function the kernels use (decode_plan.h): what
// every CTA of a launch would be given.  For tests; nothing on the product path calls it.
#include <string.h>

#include <vector>

#include "decode_plan.h"

using namespace dfi;

#define DFI_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

template <int CL, int HEAD>
void plan_all(int* out, const std::vector<int>& cum, int longest, int shortest, int n_seqs, int n_kv, int group, int launched) {
    for (int cta = 0; cta < launched; ++cta) {
        DecodePlan plan;
        dec_plan<CL, HEAD>(&plan, cum.data(), longest, shortest, n_seqs, n_kv, group, launched, cta);
        plan.reserved[0] = plan.reserved[1] = 0;
        memcpy(out + (size_t)cta * (sizeof(DecodePlan) / sizeof(int)), &plan, sizeof(DecodePlan));
    }
}

// HEAD only says whether the CTAs of a cluster can share a head's columns in fours: 128 does for every cluster
// size, a head of CL columns for none.
template <int CL>
void plan_for(bool merges, int* out, const std::vector<int>& cum, int longest, int shortest, int n_seqs, int n_kv, int group,
              int launched) {
    if (merges) plan_all<CL, 128>(out, cum, longest, shortest, n_seqs, n_kv, group, launched);
    else plan_all<CL, CL>(out, cum, longest, shortest, n_seqs, n_kv, group, launched);
}

}  // namespace

// Ints of one CTA's plan in `out`: total, n_ctas, parts, tiles, whole, uneven, group_cost, first_unit, end_unit,
// first_seq, and two that mean nothing.
DFI_EXPORT int dfi_decode_plan_ints() { return (int)(sizeof(DecodePlan) / sizeof(int)); }

// seq_start[i]: keys that sequence i holds before the step's token.  cluster: CTAs per cluster of the launch
// (1, 2, 4, 8, 16).  Returns 0, or -1 for arguments that no launch has.
DFI_EXPORT int dfi_decode_plan_host(int* out, const int* seq_start, int n_seqs, int n_kv, int group, int window, int launched,
                                    int cluster, int head_dim) {
    if (out == nullptr || seq_start == nullptr || n_seqs <= 0 || n_kv <= 0 || group <= 0 || launched <= 0 || head_dim <= 0)
        return -1;
    std::vector<int> cum(n_seqs + 1, 0);
    int longest = 0, shortest = 0x7fffffff;
    for (int i = 0; i < n_seqs; ++i) {
        const int pos = seq_start[i];
        const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
        const int tiles = pos / kPage - first_key / kPage + 1;
        cum[i + 1] = cum[i] + tiles;
        longest = max(longest, tiles);
        shortest = min(shortest, tiles);
    }
    const bool merges = cluster > 1 && head_dim % cluster == 0 && (head_dim / cluster) % 4 == 0;
    switch (cluster) {
        case 1: plan_for<1>(false, out, cum, longest, shortest, n_seqs, n_kv, group, launched); break;
        case 2: plan_for<2>(merges, out, cum, longest, shortest, n_seqs, n_kv, group, launched); break;
        case 4: plan_for<4>(merges, out, cum, longest, shortest, n_seqs, n_kv, group, launched); break;
        case 8: plan_for<8>(merges, out, cum, longest, shortest, n_seqs, n_kv, group, launched); break;
        case 16: plan_for<16>(merges, out, cum, longest, shortest, n_seqs, n_kv, group, launched); break;
        default: return -1;
    }
    return 0;
}
