// How the decode attention kernel deals the pages of a step to its CTAs: the numbers and the function that
// work it out, apart from the kernel so that the same code also compiles for the host, where tests check what
// no result on a device can show directly (every page dealt once, no group spread over more CTAs than the
// merge takes, nothing for a CTA past the last).  The kernel's file says what a CTA does with its share.
#pragma once

#if defined(__CUDACC__)
#define DFI_PLAN_HD __host__ __device__
#define DFI_PLAN_FN __host__ __device__ __forceinline__
#define DFI_PLAN_NOINLINE __noinline__
#else
#include <algorithm>
#define DFI_PLAN_HD
#define DFI_PLAN_FN inline
#define DFI_PLAN_NOINLINE __attribute__((noinline))
#endif

namespace dfi {

#if !defined(__CUDACC__)
using std::max;
using std::min;
#endif

constexpr int kPage = 64;               // keys per tile = tokens per cache page
constexpr int kDecodeCluster = 4;       // CTAs per cluster when the launch uses clusters
constexpr int kDecodeClusterWide = 8;   // ... or eight, when the groups are few and small (up to four query heads each)
constexpr int kDecodeClusterPair = 2;   // ... or two, when there are too many groups for four CTAs each
constexpr int kDecodeClusterFull = 16;  // ... or sixteen (the most a launch may ask for), for the groups of one sequence
constexpr int kFullLeastKeys = 2048;    // a launch whose sequences cannot outgrow this many keys gains nothing from sixteen
constexpr int kGroupCost = 4;           // what a group costs a CTA that touches it besides its pages, in pages
constexpr int kCutCost = 12;            // what a group cut by the end of an equal run costs, in pages of a CTA's time
constexpr int kWideMostPages = 80;      // a group of more pages than this is cut into more than eight parts
constexpr int kPartMostPages = kWideMostPages / kDecodeClusterWide;       // (so: ten pages a part in the cluster)
DFI_PLAN_HD constexpr int dec_cluster_rows(int cl) { return cl >= 8 ? 4 : 8; }
constexpr int kMaxGroupParts = 64;      // CTAs that may share one (sequence, head) group

struct DecodeRun {
    int total;      // units of the whole step
    int n_ctas;
    int parts;      // > 0: every group has `tiles` pages and is cut into this many parts, one CTA each
    int tiles;
    int whole;      // > 0: every group has `tiles` pages, there are this many groups, and a CTA takes whole groups
    int uneven;     // with parts > 0: the groups differ in length; each is cut into `parts` parts of its own pages
    int group_cost; // equal runs: units that stand for a group's fixed cost in front of its pages (see dec_plan)
};
// First unit of a CTA's run: equal contiguous runs over all units, or (when every sequence brings
// the same number of pages) the same number of parts for every group, so that no run crosses from
// one group into the next, or (many short groups) whole groups only, so that nothing is merged.
DFI_PLAN_FN int dec_run_begin(const DecodeRun& r, int cta) {
    if (r.whole > 0) {
        if (cta >= r.n_ctas) return r.total;
        return (int)((long long)r.whole * cta / r.n_ctas) * r.tiles;
    }
    if (r.parts > 0) {
        if (cta >= r.n_ctas) return r.total;
        return (cta / r.parts) * r.tiles + r.tiles * (cta % r.parts) / r.parts;
    }
    return (int)((unsigned long long)r.total * (unsigned)cta / (unsigned)r.n_ctas);
}
DFI_PLAN_FN int dec_cta_of_unit(const DecodeRun& r, int u) {
    int c;
    if (r.whole > 0) c = (int)((long long)(u / r.tiles) * r.n_ctas / r.whole);
    else if (r.parts > 0) c = (u / r.tiles) * r.parts + min(r.parts - 1, (u % r.tiles) * r.parts / r.tiles);
    else c = (int)((unsigned long long)u * (unsigned)r.n_ctas / (unsigned)r.total);
    while (c + 1 < r.n_ctas && dec_run_begin(r, c + 1) <= u) ++c;
    while (c > 0 && dec_run_begin(r, c) > u) --c;
    return c;
}

// How a launch deals its pages, and what this CTA gets: worked out by one thread of the CTA (in a function of
// its own, so that its divisions and branches stay out of the registers and the schedule of the page loop) and
// handed to the others through shared memory.
struct alignas(16) DecodePlan {
    DecodeRun run;
    int first_unit, end_unit, first_seq;
    int reserved[2];
};
static_assert(sizeof(DecodePlan) == 48, "a CTA reads its plan as three 16-byte words");
template <int CL, int HEAD>
DFI_PLAN_HD DFI_PLAN_NOINLINE void dec_plan(DecodePlan* plan, const int* cum_s, int longest, int shortest, int n_seqs, int n_kv,
                                      int group, int launched, int cta) {
    constexpr int cluster_size = CL;
    constexpr bool kClusterMerge = CL > 1 && (HEAD / (CL > 1 ? CL : 1)) % 4 == 0;
    // CTAs that the plan may give pages to.  A launch in clusters runs fewer CTAs at once than the occupancy
    // calculation promises (measured on a B200: 284 promised for clusters of four, the kernel at full speed up to
    // 272 CTAs with pages and a quarter slower from 280 on, when the last clusters wait for a place), so a
    // sixteenth of the launch is left without pages.
    // (at least one cluster: a launch of sixteen CTAs in one cluster of sixteen would otherwise be left with none)
    const int grid = CL > 1 ? max(CL, (launched - launched / 16) / CL * CL) : launched;
    DecodeRun run;
    // Equal runs are dealt in units of which every group brings kGroupCost more than it has pages: a CTA pays
    // for every group it touches (its queries prepared, the page ring started, a result stored) about what
    // that many pages cost, and a run of pages alone would hand one CTA dozens of one-page groups where they
    // lie side by side (measured: 24 sequences of 4,096 keys took 66 us, with 8 of one key beside them 130 us).
    run.group_cost = kGroupCost;
    run.total = (cum_s[n_seqs] + n_seqs * kGroupCost) * n_kv;
    // A CTA takes at least four units, and enough of them that no sequence is spread over more than
    // kMaxGroupParts CTAs.
    const int least = max(4, (longest + kGroupCost + kMaxGroupParts - 3) / (kMaxGroupParts - 2));
    run.n_ctas = max(1, min(grid, run.total / least));
    const int equal_share = run.total / run.n_ctas + kCutCost;      // what the busiest CTA of equal runs costs, in pages
    run.parts = 0;
    run.whole = 0;
    run.uneven = 0;
    run.tiles = longest;
    if (shortest == longest) {
        // every group has the same number of pages: the same number of parts for each, none crossing over
        // (as many as there are CTAs for, none shorter than the least a CTA takes)
        int parts = max(1, min(grid / (n_seqs * n_kv), longest / least));
        // Short groups with CTAs to spare: four parts each, although that leaves a CTA fewer than four pages.
        // Four parts meet in a cluster, which costs less than the pages saved (at batch 1 and 8 with some 700
        // keys a sequence the kernel took 20 us with two parts of five or six pages that met through scratch
        // memory and a ticket).
        if (parts < kDecodeCluster && longest >= kDecodeCluster && cluster_size == kDecodeCluster &&
            n_seqs * n_kv * kDecodeCluster <= grid)
            parts = kDecodeCluster;
        // A launch in clusters of eight or sixteen (few groups of up to four query heads): that many parts each,
        // as long as a part stays at ten pages or fewer, so that they meet in the cluster and not through
        // scratch memory and a ticket.
        bool by_cluster = false;          // fewer CTAs than equal runs would use, on purpose
        if (cluster_size >= kDecodeClusterWide && longest >= cluster_size && longest <= kPartMostPages * cluster_size &&
            n_seqs * n_kv * cluster_size <= grid) {
            parts = cluster_size;
            by_cluster = true;
        }
        // (not if there are more parts than CTAs, nor if they keep fewer than 80 % of the CTAs busy and a part is
        // longer than the busiest CTA of equal runs would be, cuts included: then those runs are used)
        // (sequences of one length at 80 % of the CTAs or more were measured faster cut like this than in equal
        // runs at every length: eight sequences of 32,768 keys 7.6 against 9.4 ms a step)
        if (n_seqs * n_kv * parts <= grid && (by_cluster || n_seqs * n_kv * parts * 100 >= run.n_ctas * 80 ||
                                              (longest + parts - 1) / parts + kGroupCost <= equal_share)) {
            run.parts = parts;
            run.n_ctas = n_seqs * n_kv * parts;
        } else if (n_seqs * n_kv >= grid) {
            // more groups than CTAs (many short sequences): equal runs would cut most groups in two, and every
            // cut costs a preparation of the queries, two stores of partial results, a ticket and a merge,
            // about three pages' worth of time.  Whole groups per CTA cost the busiest CTA a few pages more.
            const int groups = n_seqs * n_kv;
            const int busiest = (groups + grid - 1) / grid;
            if (busiest * (longest + kGroupCost) <= equal_share) {
                run.whole = groups;
                run.n_ctas = grid;
            }
        }
    }
    else if (const int many = max(1, min(grid / (n_seqs * n_kv), longest / least));
             many > cluster_size && shortest >= many && n_seqs * n_kv * many <= grid &&
             (longest + many - 1) / many + kGroupCost <= equal_share) {
        // Sequences of different lengths, none shorter than the number of parts that sequences of the longest's
        // length would be cut into: every group in that many parts of its own pages, which meet through scratch
        // memory and a ticket (more and shorter parts than a cluster has CTAs: the few groups of a small batch)
        run.parts = many;
        run.uneven = 1;
        run.n_ctas = n_seqs * n_kv * many;
    }
    else if (kClusterMerge && n_seqs * n_kv * cluster_size <= grid && group <= dec_cluster_rows(cluster_size)) {
        // Sequences of different lengths and few groups: every group is cut into as many parts as a cluster has
        // CTAs, each part a share of its own group's pages (none, for a group with fewer pages than parts), and
        // the parts meet in the cluster.  The CTAs of the longest sequence then hold more pages than an equal
        // share; equal runs over all pages instead cut groups wherever a run ends, and every cut costs a second
        // preparation of queries, a second start of the page ring, partial results through scratch memory and a
        // ticket: about kCutCost pages' worth (batch 8 near 3,900 keys: 3.42 ms a step with equal runs, 2.85 ms
        // with sequences of one length).
        const int per_part = (longest + cluster_size - 1) / cluster_size + kGroupCost;
        if (per_part <= equal_share) {
            run.parts = cluster_size;
            run.uneven = 1;
            run.n_ctas = n_seqs * n_kv * cluster_size;
        }
    }
    // The same with whole groups, one a CTA, where there are too many groups to cut each (and no more than CTAs):
    // nothing is merged, and the longest group is the kernel's length.
    if (shortest != longest && run.parts == 0 && n_seqs * n_kv <= grid && longest + kGroupCost <= equal_share) {
        run.parts = 1;
        run.uneven = 1;
        run.n_ctas = n_seqs * n_kv;
    }
    // More groups than CTAs: the same number of whole groups for every CTA (one more for some), if the busiest
    // CTA's pages stay within the cost of the cuts that equal runs would make.
    if (shortest != longest && run.parts == 0 && n_seqs * n_kv > grid) {
        const int groups = n_seqs * n_kv;
        const int busiest = (groups + grid - 1) / grid;
        if (busiest * (longest + kGroupCost) <= equal_share) {
            run.whole = groups;
            run.uneven = 1;
            run.n_ctas = grid;
        }
    }
    if (run.parts > 0 || run.whole > 0) {
        run.group_cost = 0;                     // groups are cut or kept one by one: the units are their pages
        run.total = cum_s[n_seqs] * n_kv;
    }
    const bool idle = cta >= run.n_ctas;
    // this CTA's units and the sequence that holds the first of them
    int first_unit = 0, end_unit = 0, first_seq = 0;
    if (idle) {
    } else if (run.uneven && run.whole > 0) {
        // whole groups g_a .. g_b - 1 of different lengths: from the first unit of the one to that of the other
        const int g_a = (int)((long long)cta * run.whole / run.n_ctas), g_b = (int)((long long)(cta + 1) * run.whole / run.n_ctas);
        first_seq = g_a / n_kv;
        first_unit = cum_s[first_seq] * n_kv + (g_a % n_kv) * (cum_s[first_seq + 1] - cum_s[first_seq]);
        const int seq_b = g_b / n_kv;
        end_unit = g_b >= run.whole ? run.total : cum_s[seq_b] * n_kv + (g_b % n_kv) * (cum_s[seq_b + 1] - cum_s[seq_b]);
    } else if (run.uneven) {
        // part `cta % parts` of group `cta / parts`: a share of that group's own pages (it may be empty)
        const int gi = cta / run.parts, part = cta % run.parts;
        first_seq = gi / n_kv;
        const int seq_tiles = cum_s[first_seq + 1] - cum_s[first_seq];
        const int first = cum_s[first_seq] * n_kv + (gi % n_kv) * seq_tiles;
        first_unit = first + seq_tiles * part / run.parts;
        end_unit = first + seq_tiles * (part + 1) / run.parts;
    } else {
        first_unit = dec_run_begin(run, cta);
        end_unit = dec_run_begin(run, cta + 1);
        // the last sequence whose first unit is not past first_unit
        int lo = 0, hi = n_seqs - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if ((cum_s[mid] + mid * run.group_cost) * n_kv <= first_unit) lo = mid; else hi = mid - 1;
        }
        first_seq = lo;
    }
    plan->run = run;
    plan->first_unit = first_unit;
    plan->end_unit = end_unit;
    plan->first_seq = first_seq;
}

}  // namespace dfi
