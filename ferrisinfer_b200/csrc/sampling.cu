// Sampling from fp32 logits: greedy, and temperature with top-k / top-p, a cluster of eight CTAs per row.
//
// The reference's sampler (crates/ferrisinfer-runtime/src/sampler.rs:77-241):
//   greedy if temperature <= 0, top_k == 1 or top_p <= 0: argmax, probability 1 / sum exp(l - max);
//   else keep the top_k largest logits, sort them descending, w = exp(l/T - max/T) with
//   T = max(T, f32 epsilon), keep the shortest prefix whose mass reaches top_p * total, draw
//   u in [0,1) from xorshift64*, threshold = u * retained_total, walk the prefix subtracting
//   weights until the threshold is <= 0; probability = w / retained_total.
//
// A walk over sorted candidates is a weighted quantile: the chosen token is the one at which the
// mass of everything before it (in descending order) first reaches the threshold.  This kernel
// finds such quantiles without sorting.  Elements are ordered by 64-bit keys (order-preserving
// logit bits, then the inverted index, so that keys are unique and ties go to the lower index).
// One histogram of 2,048 bins, LINEAR in the logit between the row's least and greatest value
// (so that a row of 150,000 logits leaves a few hundred in its fullest bin), is shared by top-k (a
// count quantile), top-p and the final draw (mass quantiles): a scan finds the bin of a quantile,
// the bin's elements are gathered into shared memory (at most 1,024) and the one element is found
// there by counting, for each, what lies before it.  A bin with more elements (many equal logits)
// is worked off by descending a radix tree over the digits of their keys instead.  Masses are
// 2^-40 fixed-point integers: sums are exact and independent of the order of the atomic
// additions, so the result is deterministic.
//
// The eight CTAs of a row each read an eighth of the vocabulary in every pass; their histograms are added through
// the cluster's shared memory (every CTA reads all eight and keeps the totals, so all take the same decisions
// without a broadcast), and whoever finds the one element of a leaf tells the others the same way.
//
// RNG: one xorshift64* state per request slot, advanced once per sampled (non-greedy) token
// (crates/ferrisinfer-runtime/src/sampler.rs:50-75), so a request's draws do not depend on what
// else is in the batch.
#include <float.h>
#include <math.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 1024;
constexpr int BINS = 2048;
constexpr int NUM_DIGITS = 6;
__device__ __constant__ int kShift[NUM_DIGITS] = {53, 42, 31, 20, 9, 0};
__device__ __constant__ int kWidth[NUM_DIGITS] = {11, 11, 11, 11, 11, 9};

typedef unsigned long long u64;
typedef unsigned int u32;

// barrier over all threads of all CTAs of the cluster; an fp32 from CTA `rank`'s shared memory
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float peer_shared_f32(u32 addr, u32 rank) {
    u32 remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

__device__ __forceinline__ u32 peer_shared_u32(u32 addr, u32 rank) {
    u32 remote, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ u64 peer_shared_u64(u32 addr, u32 rank) {
    u32 remote;
    u64 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote) : "memory");
    return v;
}

constexpr int ROW_CLUSTER = 8;  // CTAs per row
constexpr int LIST_CAP = 1024;  // elements of one bin that are gathered and searched in shared memory

__device__ __forceinline__ u64 make_key(float logit, int index) {
    u32 u = __float_as_uint(logit);
    u32 k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    if (logit != logit) k = 0;  // NaN sorts last
    return ((u64)k << 32) | (u64)(0xFFFFFFFFu - (u32)index);
}

struct Shared {
    u32 count[BINS];
    u64 mass[BINS];
    u64 warp_count[32];
    u64 warp_mass[32];
    u64 red[32];
    // results of a scan / find
    int chosen_bin;
    u32 chosen_count;
    u64 excl_count, excl_mass;
    u64 found_key, found_mass;
    u32 found;         // 1 if this CTA's part of the row holds the element that find_unique looked for
    u64 best_key;      // this CTA's greatest key
    float part_denom;  // this CTA's part of a greedy row's sum of exponentials
    float part_min;    // this CTA's least finite logit
    // the elements of one bin: this CTA's, and the whole row's
    u32 own_count;
    u64 own_key[LIST_CAP], own_mass[LIST_CAP];
    u64 all_key[LIST_CAP], all_mass[LIST_CAP];
    u64 before_mass;   // mass before the element that select_in_list found
    // level-0 histogram kept for the later descents
    u32 count0[BINS];
    u64 mass0[BINS];
};

struct RowArgs {
    const float* row;
    int V;
    int lo, hi;  // this CTA's part of the row
    float inv_t_max;  // max / T
    float T;
    float top;        // the row's greatest logit
    float lin_scale;  // bins per unit of logit of the linear histogram
};

// The bin of the linear histogram: the greatest logits in the highest bin, monotone in the logit; everything below
// the histogram's range (and a NaN) in bin 0.
__device__ __forceinline__ int linear_bin(const RowArgs& a, float l) {
    const float x = l == a.top ? 0.0f : (a.top - l) * a.lin_scale;
    return BINS - 1 - (int)fminf(x, (float)(BINS - 1));  // fminf(NaN, c) = c
}

__device__ __forceinline__ u64 weight_fixed(const RowArgs& a, float logit) {
    const float w = expf(logit / a.T - a.inv_t_max);
    return (u64)((double)w * 1099511627776.0);  // 2^40; w <= 1
}

// f(logit, index) for every element of this CTA's part of the row, each thread its share; four at a time (one
// 16-byte load) where the part begins on a 16-byte boundary.
template <typename F>
__device__ __forceinline__ void for_slice(const RowArgs& a, F f) {
    if ((reinterpret_cast<uintptr_t>(a.row + a.lo) & 15) == 0) {
        const int whole = a.lo + ((a.hi - a.lo) & ~3);
        for (int i = a.lo + 4 * (int)threadIdx.x; i < whole; i += 4 * THREADS) {
            const float4 v = *reinterpret_cast<const float4*>(a.row + i);
            f(v.x, i);
            f(v.y, i + 1);
            f(v.z, i + 2);
            f(v.w, i + 3);
        }
        for (int i = whole + (int)threadIdx.x; i < a.hi; i += THREADS) f(a.row[i], i);
    } else {
        for (int i = a.lo + (int)threadIdx.x; i < a.hi; i += THREADS) f(a.row[i], i);
    }
}

// d < 0: the linear histogram of the whole row.  Otherwise: the histogram of key digit d over the elements of bin
// `lin_bin` of the linear histogram whose higher key digits equal those of `prefix`.
__device__ void hist_pass(Shared& s, const RowArgs& a, int lin_bin, u64 prefix, int d) {
    for (int b = threadIdx.x; b < BINS; b += THREADS) {
        s.count[b] = 0;
        s.mass[b] = 0;
    }
    __syncthreads();
    const int shift = d >= 0 ? kShift[d] : 0;
    const u32 mask = d >= 0 ? (1u << kWidth[d]) - 1u : 0u;
    const int up = d > 0 ? kShift[d - 1] : 64;
    // a small per-thread cache of buckets, so that clustered logits do not serialise on one counter
    int cb0 = -1, cb1 = -1, cb2 = -1, cb3 = -1;
    u32 cc0 = 0, cc1 = 0, cc2 = 0, cc3 = 0;
    u64 cm0 = 0, cm1 = 0, cm2 = 0, cm3 = 0;
    int victim = 0;
    for_slice(a, [&](float l, int i) {
        const u64 key = make_key(l, i);
        const int lb = linear_bin(a, l);
        if (d >= 0 && lb != lin_bin) return;
        if (d > 0 && (key >> up) != (prefix >> up)) return;
        const int b = d >= 0 ? (int)((key >> shift) & mask) : lb;
        const u64 m = weight_fixed(a, l);
        if (b == cb0) { cc0++; cm0 += m; }
        else if (b == cb1) { cc1++; cm1 += m; }
        else if (b == cb2) { cc2++; cm2 += m; }
        else if (b == cb3) { cc3++; cm3 += m; }
        else {
            int ob; u32 oc; u64 om;
            if (victim == 0) { ob = cb0; oc = cc0; om = cm0; cb0 = b; cc0 = 1; cm0 = m; }
            else if (victim == 1) { ob = cb1; oc = cc1; om = cm1; cb1 = b; cc1 = 1; cm1 = m; }
            else if (victim == 2) { ob = cb2; oc = cc2; om = cm2; cb2 = b; cc2 = 1; cm2 = m; }
            else { ob = cb3; oc = cc3; om = cm3; cb3 = b; cc3 = 1; cm3 = m; }
            victim = (victim + 1) & 3;
            if (ob >= 0) {
                atomicAdd(&s.count[ob], oc);
                atomicAdd(&s.mass[ob], om);
            }
        }
    });
    if (cb0 >= 0) { atomicAdd(&s.count[cb0], cc0); atomicAdd(&s.mass[cb0], cm0); }
    if (cb1 >= 0) { atomicAdd(&s.count[cb1], cc1); atomicAdd(&s.mass[cb1], cm1); }
    if (cb2 >= 0) { atomicAdd(&s.count[cb2], cc2); atomicAdd(&s.mass[cb2], cm2); }
    if (cb3 >= 0) { atomicAdd(&s.count[cb3], cc3); atomicAdd(&s.mass[cb3], cm3); }
    __syncthreads();
}

// The histograms of the row's CTAs (s.count / s.mass of each) added up into `count` / `mass` of this CTA: every CTA
// reads all of them in rank order and ends with the same totals.  `count` / `mass` may be s.count / s.mass themselves
// (a thread replaces only the bins it has read from every CTA, after the cluster's second barrier).
__device__ void merge_hist(Shared& s, u32* count, u64* mass) {
    cluster_sync_all();  // every CTA's histogram is complete
    u32 c[BINS / THREADS];
    u64 m[BINS / THREADS];
#pragma unroll
    for (int j = 0; j < BINS / THREADS; ++j) {
        const int b = threadIdx.x + j * THREADS;
        const u32 ca = (u32)__cvta_generic_to_shared(&s.count[b]), ma = (u32)__cvta_generic_to_shared(&s.mass[b]);
        u32 pc[ROW_CLUSTER];
        u64 pm[ROW_CLUSTER];
#pragma unroll
        for (int r = 0; r < ROW_CLUSTER; ++r) {
            pc[r] = peer_shared_u32(ca, r);
            pm[r] = peer_shared_u64(ma, r);
        }
        c[j] = 0;
        m[j] = 0;
#pragma unroll
        for (int r = 0; r < ROW_CLUSTER; ++r) {
            c[j] += pc[r];
            m[j] += pm[r];
        }
    }
    cluster_sync_all();  // nobody's histogram is read any more
#pragma unroll
    for (int j = 0; j < BINS / THREADS; ++j) {
        count[threadIdx.x + j * THREADS] = c[j];
        mass[threadIdx.x + j * THREADS] = m[j];
    }
    __syncthreads();
}

// Scan the histogram from the highest bin down; pick the bin in which the running total
// (of counts if by_count, else of masses) first reaches `target`.
__device__ void scan_pick(Shared& s, const u32* count, const u64* mass, bool by_count, u64 target) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // thread t owns descending bins 2t, 2t+1 -> actual bins BINS-1-2t, BINS-2-2t
    const int b0 = BINS - 1 - 2 * threadIdx.x, b1 = b0 - 1;
    const u64 c0 = count[b0], c1 = count[b1];
    const u64 m0 = mass[b0], m1 = mass[b1];
    u64 pc = c0 + c1, pm = m0 + m1;  // inclusive scan within the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 tc = __shfl_up_sync(0xffffffffu, pc, o);
        const u64 tm = __shfl_up_sync(0xffffffffu, pm, o);
        if (lane >= o) { pc += tc; pm += tm; }
    }
    if (lane == 31) { s.warp_count[warp] = pc; s.warp_mass[warp] = pm; }
    if (threadIdx.x == 0) { s.chosen_bin = -1; }
    __syncthreads();
    u64 oc = 0, om = 0;
    for (int w = 0; w < warp; ++w) { oc += s.warp_count[w]; om += s.warp_mass[w]; }
    const u64 incl_c = oc + pc, incl_m = om + pm;
    const u64 excl_c = incl_c - (c0 + c1), excl_m = incl_m - (m0 + m1);
    // first bin of the pair
    {
        const u64 before = by_count ? excl_c : excl_m;
        const u64 after = by_count ? excl_c + c0 : excl_m + m0;
        if (c0 > 0 && before < target && target <= after) {
            s.chosen_bin = b0; s.chosen_count = (u32)c0; s.excl_count = excl_c; s.excl_mass = excl_m;
        }
    }
    {
        const u64 before = by_count ? excl_c + c0 : excl_m + m0;
        const u64 after = by_count ? incl_c : incl_m;
        if (c1 > 0 && before < target && target <= after) {
            s.chosen_bin = b1; s.chosen_count = (u32)c1; s.excl_count = excl_c + c0; s.excl_mass = excl_m + m0;
        }
    }
    __syncthreads();
    if (s.chosen_bin < 0) {
        // the target lies beyond the total (only possible through the caller's rounding): take the
        // lowest bin that holds anything
        if (threadIdx.x == 0) {
            u64 ec = 0, em = 0;
            int last = -1;
            for (int b = BINS - 1; b >= 0; --b)
                if (count[b]) last = b;
            for (int b = BINS - 1; b > last; --b) { ec += count[b]; em += mass[b]; }
            s.chosen_bin = last; s.chosen_count = count[last]; s.excl_count = ec; s.excl_mass = em;
        }
        __syncthreads();
    }
}

// The only element whose digits 0..d equal those of `prefix`.
__device__ void find_unique(Shared& s, const RowArgs& a, int lin_bin, u64 prefix, int d) {
    const int shift = kShift[d];
    if (threadIdx.x == 0) s.found = 0;
    __syncthreads();
    for_slice(a, [&](float l, int i) {
        const u64 key = make_key(l, i);
        if (linear_bin(a, l) == lin_bin && (key >> shift) == (prefix >> shift)) {
            s.found_key = key;
            s.found_mass = weight_fixed(a, l);
            s.found = 1;
        }
    });
    __syncthreads();
    // the CTA whose part of the row holds it tells the others
    cluster_sync_all();
    u64 key = 0, mass = 0;
    if (threadIdx.x == 0) {
        const u32 fa = (u32)__cvta_generic_to_shared(&s.found), ka = (u32)__cvta_generic_to_shared(&s.found_key),
                  ma = (u32)__cvta_generic_to_shared(&s.found_mass);
        for (int r = 0; r < ROW_CLUSTER; ++r)
            if (peer_shared_u32(fa, r)) {
                key = peer_shared_u64(ka, r);
                mass = peer_shared_u64(ma, r);
            }
    }
    cluster_sync_all();  // everyone has read
    if (threadIdx.x == 0) {
        s.found_key = key;
        s.found_mass = mass;
    }
    __syncthreads();
}


// The `n` elements of bin `lin_bin` (n <= LIST_CAP) from every CTA's part of the row into s.all_key / s.all_mass of
// every CTA, in the order of the CTAs.
__device__ void gather_bin(Shared& s, const RowArgs& a, int lin_bin) {
    if (threadIdx.x == 0) s.own_count = 0;
    __syncthreads();
    for_slice(a, [&](float l, int i) {
        if (linear_bin(a, l) != lin_bin) return;
        const u32 at = atomicAdd(&s.own_count, 1u);
        if (at < LIST_CAP) {
            s.own_key[at] = make_key(l, i);
            s.own_mass[at] = weight_fixed(a, l);
        }
    });
    __syncthreads();
    cluster_sync_all();
    const u32 ca = (u32)__cvta_generic_to_shared(&s.own_count);
    u32 offset = 0;
    for (int r = 0; r < ROW_CLUSTER; ++r) {
        const u32 n = peer_shared_u32(ca, r);
        for (u32 j = threadIdx.x; j < n && offset + j < LIST_CAP; j += THREADS) {
            s.all_key[offset + j] = peer_shared_u64((u32)__cvta_generic_to_shared(&s.own_key[j]), r);
            s.all_mass[offset + j] = peer_shared_u64((u32)__cvta_generic_to_shared(&s.own_mass[j]), r);
        }
        offset += n;
    }
    cluster_sync_all();  // the lists are complete everywhere, and nobody's own list is read any more
}

// Among the n gathered elements: the one at which the running total (of counts if by_count, else of masses), taken
// in descending key order, first reaches `target`; the lowest key if the target lies beyond the total (only
// possible through the caller's rounding).  Leaves it in s.found_key / s.found_mass, the mass before it in s.before_mass.
__device__ void select_in_list(Shared& s, int n, bool by_count, u64 target) {
    if (threadIdx.x == 0) s.found = 0;
    __syncthreads();
    u64 key = 0, mass = 0, before_m = 0;
    u32 before_c = 0;
    const bool mine = (int)threadIdx.x < n;
    if (mine) {
        key = s.all_key[threadIdx.x];
        mass = s.all_mass[threadIdx.x];
        for (int j = 0; j < n; ++j) {
            const u64 kj = s.all_key[j];
            if (kj > key) {
                ++before_c;
                before_m += s.all_mass[j];
            }
        }
        const bool hit = by_count ? ((u64)before_c < target && target <= (u64)before_c + 1)
                                  : (before_m < target && target <= before_m + mass);
        if (hit) {
            s.found_key = key;
            s.found_mass = mass;
            s.before_mass = before_m;
            s.found = 1;
        }
    }
    __syncthreads();
    if (!s.found && mine && (int)before_c == n - 1) {
        s.found_key = key;
        s.found_mass = mass;
        s.before_mass = before_m;
    }
    __syncthreads();
}

struct Quantile {
    u64 key;       // the element at which the running total first reaches the target
    u64 mass_ge;   // mass of all elements with key >= key
    u64 mass_self; // its own mass
};

// The quantile from the row's linear histogram (count0 / mass0, the same in every CTA of the row).
__device__ Quantile descend(Shared& s, const RowArgs& a, bool by_count, u64 target) {
    Quantile q;
    scan_pick(s, s.count0, s.mass0, by_count, target);
    const int lin_bin = s.chosen_bin;
    const u32 in_bin = s.chosen_count;
    u64 cum_mass = s.excl_mass;
    target -= by_count ? s.excl_count : s.excl_mass;
    __syncthreads();
    if (in_bin <= LIST_CAP) {
        gather_bin(s, a, lin_bin);
        select_in_list(s, (int)in_bin, by_count, target);
        q.key = s.found_key;
        q.mass_self = s.found_mass;
        q.mass_ge = cum_mass + s.before_mass + s.found_mass;
        __syncthreads();
        return q;
    }
    // many elements in one bin: a radix tree over the digits of their keys
    u64 prefix = 0;
    for (int d = 0; d < NUM_DIGITS; ++d) {
        hist_pass(s, a, lin_bin, prefix, d);
        merge_hist(s, s.count, s.mass);
        scan_pick(s, s.count, s.mass, by_count, target);
        const int bin = s.chosen_bin;
        const u32 cnt = s.chosen_count;
        const u64 ec = s.excl_count, em = s.excl_mass;
        __syncthreads();
        cum_mass += em;
        target -= by_count ? ec : em;
        prefix |= (u64)bin << kShift[d];
        if (cnt == 1 || d == NUM_DIGITS - 1) {
            find_unique(s, a, lin_bin, prefix, d);
            q.key = s.found_key;
            q.mass_self = s.found_mass;
            q.mass_ge = cum_mass + s.found_mass;
            __syncthreads();
            return q;
        }
    }
    return q;  // not reached
}

__device__ __forceinline__ u64 block_max_u64(u64 v, u64* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const u64 t = __shfl_xor_sync(0xffffffffu, v, o);
        v = t > v ? t : v;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    u64 r = red[0];
    for (int w = 1; w < THREADS / 32; ++w) r = red[w] > r ? red[w] : r;
    __syncthreads();
    return r;
}

// Maximum over the block; every thread gets it.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_max_f32(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = scratch[0];
    for (int w = 1; w < THREADS / 32; ++w) r = fmaxf(r, scratch[w]);
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(THREADS)
    sample_kernel(const float* logits, int ldl, int V, const float* __restrict__ temperature,
                  const int* __restrict__ top_k, const float* __restrict__ top_p, const int* __restrict__ slots,
                  u64* __restrict__ rng_states, int* __restrict__ out_token, float* __restrict__ out_prob) {
    extern __shared__ __align__(16) unsigned char raw[];
    Shared& s = *reinterpret_cast<Shared*>(raw);
    __shared__ float fscratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int rank = (int)(blockIdx.z % ROW_CLUSTER);
    const float* row = logits + (size_t)r * ldl;
    const float T = temperature ? temperature[r] : 0.0f;
    const int k = top_k ? top_k[r] : 0;
    const float p = top_p ? top_p[r] : 1.0f;
    const bool greedy = !(T > 0.0f) || k == 1 || !(p > 0.0f);
    // the generator's state is read by every CTA of the row now and advanced by the first one much later, after
    // barriers of the cluster
    const u64 rng_before = (!greedy && threadIdx.x == 0) ? rng_states[slots[r]] : 0;
    const int per = ((V + 4 * ROW_CLUSTER - 1) / (4 * ROW_CLUSTER)) * 4;
    const int lo = min(V, rank * per), hi = min(V, lo + per);

    // argmax (lowest index among equal maxima) through the key order
    RowArgs a;
    a.row = row;
    a.V = V;
    a.lo = lo;
    a.hi = hi;
    u64 best = 0;
    float least = INFINITY;  // the least finite logit
    for_slice(a, [&](float l, int i) {
        const u64 key = make_key(l, i);
        best = key > best ? key : best;
        if (l > -INFINITY) least = fminf(least, l);
    });
    best = block_max_u64(best, s.red);
    least = -block_max_f32(-least, fscratch);
    if (threadIdx.x == 0) {
        s.best_key = best;
        s.part_min = least;
    }
    cluster_sync_all();
    {
        const u32 ba = (u32)__cvta_generic_to_shared(&s.best_key), la = (u32)__cvta_generic_to_shared(&s.part_min);
#pragma unroll
        for (int c = 0; c < ROW_CLUSTER; ++c) {
            const u64 other = peer_shared_u64(ba, c);
            best = other > best ? other : best;
            least = fminf(least, peer_shared_f32(la, c));
        }
    }
    const int best_index = (int)(0xFFFFFFFFu - (u32)(best & 0xFFFFFFFFu));
    const float max_logit = row[best_index];

    if (greedy) {
        float denom = 0.0f;
        for_slice(a, [&](float l, int) { denom += expf(l - max_logit); });
        denom = block_sum(denom, fscratch);
        if (threadIdx.x == 0) s.part_denom = denom;
        cluster_sync_all();
        if (rank == 0 && threadIdx.x == 0) {
            const u32 da = (u32)__cvta_generic_to_shared(&s.part_denom);
            float total = 0.0f;
            for (int c = 0; c < ROW_CLUSTER; ++c) total += peer_shared_f32(da, c);
            out_token[r] = best_index;
            if (out_prob) out_prob[r] = 1.0f / total;
        }
        cluster_sync_all();  // nobody leaves while the first CTA may still read its shared memory
        return;
    }

    a.T = fmaxf(T, FLT_EPSILON);
    a.inv_t_max = max_logit / a.T;
    a.top = max_logit;
    // the linear histogram spans the row's values, but no more than 100 T below the greatest: what lies lower has
    // no weight (exp(-100) in 32 bits is 0) and shares bin 0
    float range = fminf(max_logit - least, 100.0f * a.T);
    if (!(range > 0.0f) || range == INFINITY) range = 1.0f;
    a.lin_scale = (float)(BINS - 1) / range;

    hist_pass(s, a, 0, 0, -1);
    merge_hist(s, s.count0, s.mass0);  // its barriers also cover the reads of best_key and part_min above

    const int k_eff = (k <= 0 || k > V) ? V : k;
    // mass of the top-k set: the count quantile at k
    Quantile qk = descend(s, a, true, (u64)k_eff);
    const u64 total_k = qk.mass_ge;
    u64 retained = total_k;
    if (p < 1.0f) {
        u64 cutoff = (u64)((double)total_k * (double)p);
        if (cutoff < 1) cutoff = 1;
        if (cutoff > total_k) cutoff = total_k;
        Quantile qp = descend(s, a, false, cutoff);
        retained = qp.mass_ge;
    }
    // one uniform draw from the request's own generator
    __shared__ float u_shared;
    if (threadIdx.x == 0) {
        u64 x = rng_before;
        if (x == 0) x = 0x9e3779b97f4a7c15ull;
        x ^= x >> 12;
        x ^= x << 25;
        x ^= x >> 27;
        if (rank == 0) rng_states[slots[r]] = x;
        const u64 value = x * 0x2545F4914F6CDD1Dull;
        u_shared = (float)(u32)(value >> 40) / 16777216.0f;
    }
    __syncthreads();
    u64 threshold = (u64)((double)u_shared * (double)retained);
    if (threshold < 1) threshold = 1;
    if (threshold > retained) threshold = retained;
    Quantile qs = descend(s, a, false, threshold);
    if (rank == 0 && threadIdx.x == 0) {
        out_token[r] = (int)(0xFFFFFFFFu - (u32)(qs.key & 0xFFFFFFFFu));
        if (out_prob) out_prob[r] = (float)((double)qs.mass_self / (double)retained);
    }
}

// ---------------------------------------------------------------------------------------------
// Greedy rows only: a cluster of eight CTAs per row, each over an eighth of the vocabulary in ONE pass
// (the running maximum with the sum of exp(l - maximum) rescaled when the maximum moves), combined
// through the cluster's shared memory.  Same results as the general kernel's greedy branch: the lowest
// index among equal maxima, probability 1 / sum exp(l - max).
// ---------------------------------------------------------------------------------------------
constexpr int GREEDY_CLUSTER = 8;
constexpr int GREEDY_THREADS = 512;

struct OnlineMax {
    u64 best = 0;
    float m = -INFINITY, s = 0.0f;
    __device__ __forceinline__ void take(float x, int i) {
        const u64 key = make_key(x, i);
        best = key > best ? key : best;
        if (x > m) {
            s *= expf(m - x);  // exp(-inf) = 0 the first time
            m = x;
        }
        s += m == -INFINITY ? 0.0f : expf(x - m);
    }
};

__global__ void __launch_bounds__(GREEDY_THREADS)
    greedy_kernel(const float* logits, int ldl, int V, int* __restrict__ out_token,
                  float* __restrict__ out_prob) {
    __shared__ u64 red[32];
    __shared__ float fred[33];
    __shared__ float part[4];  // this CTA's result: key (two words), maximum, sum
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int r = blockIdx.x;
    const int rank = (int)(blockIdx.z % GREEDY_CLUSTER);
    const float* row = logits + (size_t)r * ldl;
    const int per = ((V + 4 * GREEDY_CLUSTER - 1) / (4 * GREEDY_CLUSTER)) * 4;
    const int lo = min(V, rank * per), hi = min(V, lo + per);
    OnlineMax acc;
    if ((reinterpret_cast<uintptr_t>(row + lo) & 15) == 0) {
        const int whole = lo + ((hi - lo) & ~3);
        for (int i = lo + 4 * (int)threadIdx.x; i < whole; i += 4 * GREEDY_THREADS) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            acc.take(v.x, i);
            acc.take(v.y, i + 1);
            acc.take(v.z, i + 2);
            acc.take(v.w, i + 3);
        }
        for (int i = whole + (int)threadIdx.x; i < hi; i += GREEDY_THREADS) acc.take(row[i], i);
    } else {
        for (int i = lo + (int)threadIdx.x; i < hi; i += GREEDY_THREADS) acc.take(row[i], i);
    }
    // block: best key, maximum, and the sums brought to that maximum
    u64 best = acc.best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const u64 t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = best;
    float m = warp_max(acc.m);
    if (lane == 0) fred[warp] = m;
    __syncthreads();
    best = red[0];
    m = fred[0];
    for (int w = 1; w < GREEDY_THREADS / 32; ++w) {
        best = red[w] > best ? red[w] : best;
        m = fmaxf(m, fred[w]);
    }
    __syncthreads();
    float sum = acc.m == -INFINITY ? 0.0f : acc.s * expf(acc.m - m);
    sum = warp_sum(sum);
    if (lane == 0) fred[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < GREEDY_THREADS / 32; ++w) total += fred[w];
        part[0] = __uint_as_float((u32)(best >> 32));
        part[1] = __uint_as_float((u32)(best & 0xFFFFFFFFu));
        part[2] = m;
        part[3] = total;
    }
    cluster_sync_all();
    if (rank == 0 && threadIdx.x == 0) {
        const u32 addr = (u32)__cvta_generic_to_shared(part);
        u64 key = 0;
        float ms[GREEDY_CLUSTER], ss[GREEDY_CLUSTER], mm = -INFINITY;
#pragma unroll
        for (int c = 0; c < GREEDY_CLUSTER; ++c) {
            const u64 k = ((u64)__float_as_uint(peer_shared_f32(addr, c)) << 32) | (u64)__float_as_uint(peer_shared_f32(addr + 4, c));
            key = k > key ? k : key;
            ms[c] = peer_shared_f32(addr + 8, c);
            ss[c] = peer_shared_f32(addr + 12, c);
            mm = fmaxf(mm, ms[c]);
        }
        float denom = 0.0f;
#pragma unroll
        for (int c = 0; c < GREEDY_CLUSTER; ++c) denom += ms[c] == -INFINITY ? 0.0f : ss[c] * expf(ms[c] - mm);
        out_token[r] = (int)(0xFFFFFFFFu - (u32)(key & 0xFFFFFFFFu));
        if (out_prob) out_prob[r] = 1.0f / denom;
    }
    cluster_sync_all();  // nobody leaves while rank 0 may still read its shared memory
    FERRIS_TL_END(5);
}

}  // namespace

// logits fp32 [rows, V] (row stride ldl).  temperature / top_k / top_p: per row, or null for greedy.
// slots[r] indexes rng_states (one u64 per request slot; 0 stands for the reference's default seed).
FERRIS_API int ferris_sample(const float* logits, int ldl, int rows, int V, const float* temperature, const int* top_k,
                             const float* top_p, const int* slots, unsigned long long* rng_states, int* out_token,
                             float* out_prob, void* stream) {
    if (rows <= 0) return FERRIS_OK;
    if (V <= 0 || ldl < V) FERRIS_REFUSE("sample: vocabulary %d, row stride %d", V, ldl);
    if (temperature && (!slots || !rng_states)) FERRIS_REFUSE("sample: sampling with a temperature needs generator states");
    if (!temperature) {
        cudaError_t e = ferris_launch_cluster(greedy_kernel, dim3(rows, 1, GREEDY_CLUSTER), dim3(GREEDY_THREADS), 0,
                                              (cudaStream_t)stream, GREEDY_CLUSTER, logits, ldl, V, out_token, out_prob);
        if (e != cudaSuccess) {
            ferris_set_error("sample: %s", cudaGetErrorString(e));
            return (int)e;
        }
        FERRIS_LAUNCH_CHECK();
    }
    static bool configured = false;
    const size_t smem = sizeof(Shared);
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            ferris_set_error("sample: %s", cudaGetErrorString(e));
            return (int)e;
        }
        configured = true;
    }
    cudaError_t e = ferris_launch_cluster(sample_kernel, dim3(rows, 1, ROW_CLUSTER), dim3(THREADS), smem, (cudaStream_t)stream,
                                          ROW_CLUSTER, logits, ldl, V, temperature, top_k, top_p, slots, rng_states, out_token,
                                          out_prob);
    if (e != cudaSuccess) {
        ferris_set_error("sample: %s", cudaGetErrorString(e));
        return (int)e;
    }
    FERRIS_LAUNCH_CHECK();
}

FERRIS_TIMELINE_TU(sampling)
