// On-device sampler: one block per live sequence slot.
//
// Follows the reference's host sampler (src/inference.cpp:101-160):
//   repetition penalty once per distinct id of the slot's whole history (:104-112),
//   greedy = first maximum (:116-119), else weights expf((s - max)/T) (:126-131),
//   candidates in descending probability (:138), the shortest prefix whose probability mass
//   reaches top_p (:141-148), a draw from the kept candidates by inverse CDF in that order
//   (std::discrete_distribution, :151-154), append, stop on EOS / stop token (:158-160).
// No sort is performed.  Probability mass is held as 64-bit fixed point (weight * 2^47, exact for
// every weight >= 2^-24), so partial sums are associative and the result is independent of the
// order in which threads add.  "The element at which the descending cumulative mass first reaches
// a target" is found by bucket refinement over the weights' float bit patterns: a 1024-bucket
// level-0 histogram (64 buckets per octave over the top 16 octaves, shared by both queries), then
// <= 3 narrower histograms per query; ties (equal weights) go to the lower id.
// Three kernels per sampling step, because one block can push only about one shared-memory atomic
// per clock and a histogram of 32768 weights on a single SM therefore costs tens of microseconds:
//   k_samp_max   (blocks_per_slot x n_slots blocks)  penalised scores, per-block first maximum
//   k_samp_hist  (same grid)  weights expf((s - max)/T) to global memory, level-0 histogram by
//                reductions in L2 (spread over all SMs and memory slices)
//   k_samp_pick  (one block per slot)  top-p cut, draw, append, stop rules, next pass inputs
// With temperature <= 0 only k_samp_max and k_samp_pick run.
#pragma once
#include "common.cuh"

namespace sllm {

constexpr int kSampThreads = 1024;
constexpr int kSampBuckets = 1024;              // buckets of a refinement histogram in shared memory
constexpr int kL0Buckets = 8192;                // buckets of the level-0 histogram in global memory
constexpr int kL0PerThread = kL0Buckets / kSampThreads;
constexpr int kFixShift = 47;

struct SeqState {                 // device arrays indexed by slot
    uint32_t* tokens;             // [max_batch][tok_cap]
    int* n_tok;                   // tokens held (prompt + continuation)
    int* finished;                // 0 live, 1 EOS/stop, 2 context exhausted, 3 non-finite logits
    uint32_t* seen;               // [max_batch][V/32] bitmap of ids in the history
    int* draw_idx;                // next entry of the slot's draw list
    int tok_cap;
};

struct SampleArgs {
    const float* logits;          // [n_slots][V] step logits
    SeqState st;
    int V, ctx;
    float temperature, top_p, penalty;
    uint32_t eos;
    long long stop_token;
    const double* draws;          // device [n_slots][draws_stride]; entry draw_idx[slot] is used
    int n_slots;
    int draws_stride;
    int seeded;                   // 0: one entry per sampling step.  1: an entry is consumed only when at least
                                  //    two candidates are kept (std::discrete_distribution's behaviour)
    // global scratch: level-0 histogram [n_slots][1024] (zero between steps), weights [n_slots][V],
    // per-block maxima [n_slots][bps]
    unsigned long long* g_mass;
    unsigned int* g_cnt;
    float* g_w;
    float* g_pmax_val;
    int* g_pmax_idx;
    int bps;                      // blocks per slot in k_samp_max / k_samp_hist
    // next-pass token list, written for the decode step that follows
    uint32_t* next_tok_id;
    int* next_tok_pos;
    int* next_tok_slot;
};

// weight in [0,1] -> floor(weight * 2^47), by integer arithmetic on the float's bits
__device__ __forceinline__ unsigned long long fix_of(float w) {
    const uint32_t b = __float_as_uint(w);
    const int e = (int)(b >> 23);
    if (e == 0) return 0ull;                                   // denormals are below 2^-47
    const unsigned long long man = (unsigned long long)((b & 0x7fffffu) | 0x800000u);
    const int sh = e - 150 + kFixShift;                        // value = man * 2^(e-150)
    if (sh >= 0) return man << sh;
    return sh > -24 ? (man >> (-sh)) : 0ull;
}

struct SampHist {                 // shared-memory histogram: mass as 16-bit limbs, plus counts
    unsigned int l0[kSampBuckets], l1[kSampBuckets], l2[kSampBuckets], cnt[kSampBuckets];
};
__device__ __forceinline__ void hist_add(SampHist& h, int b, unsigned long long q) {
    atomicAdd(&h.l0[b], (unsigned int)(q & 0xffffu));
    atomicAdd(&h.l1[b], (unsigned int)((q >> 16) & 0xffffu));
    atomicAdd(&h.l2[b], (unsigned int)(q >> 32));              // <= 2^15 per element
    atomicAdd(&h.cnt[b], 1u);
}
__device__ __forceinline__ unsigned long long hist_mass(const SampHist& h, int b) {
    return (unsigned long long)h.l0[b] + ((unsigned long long)h.l1[b] << 16) + ((unsigned long long)h.l2[b] << 32);
}
__device__ __forceinline__ void hist_clear(SampHist& h) {
    for (int b = threadIdx.x; b < kSampBuckets; b += kSampThreads) { h.l0[b] = 0; h.l1[b] = 0; h.l2[b] = 0; h.cnt[b] = 0; }
}
__device__ __forceinline__ int shift_for(uint32_t width) {
    int sh = 0;
    while ((width >> sh) >= (uint32_t)kSampBuckets) ++sh;
    return sh;
}

struct SampScratch {
    unsigned long long sc_m[32];
    unsigned int sc_c[32];
    unsigned long long pk_above_m, pk_m, tot_m;
    unsigned int pk_above_c, pk_c, tot_c;
    int pick;
};

struct SelectResult { uint32_t key; unsigned long long cum_above, qk; unsigned int cnt_above, ties, r; int found; };

// Level-0 bucket of a weight key: 512 buckets per octave, the top bucket holds 1.0, bucket 0 everything below
// 2^-16.  Narrow buckets keep the candidate lists short (tens of elements even when the distribution is flat)
// and spread the histogram's reductions over many addresses.
constexpr uint32_t kL0Shift = 14;
constexpr uint32_t kL0Top = 0x3F800000u >> kL0Shift;          // 65024
__device__ __forceinline__ int l0_bucket(uint32_t key) {
    const int b = (int)(key >> kL0Shift) - (int)(kL0Top - (kL0Buckets - 1));
    return b < 0 ? 0 : (b > kL0Buckets - 1 ? kL0Buckets - 1 : b);
}
__device__ __forceinline__ void l0_range(int b, uint32_t& lo, uint32_t& hi) {
    lo = b == 0 ? 0u : ((uint32_t)(b + (int)kL0Top - (kL0Buckets - 1)) << kL0Shift);
    hi = (((uint32_t)(b + (int)kL0Top - (kL0Buckets - 1)) + 1u) << kL0Shift) - 1u;
}

// Thread j holds bucket (top - j) of a histogram (my_m, my_c; zero when top - j < 0).  Picks the first
// non-empty bucket, scanning from the highest, at which cum + running mass reaches target.  Returns the
// picked bucket index or -1; cum / cnt absorb what lies above the pick (or everything when none is picked).
__device__ int scan_pick(unsigned long long my_m, unsigned int my_c, int top, SampScratch& s, unsigned long long target,
                         unsigned long long& cum, unsigned int& cnt, unsigned long long& bucket_mass, unsigned int& bucket_cnt) {
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const int b = top - tid;
    unsigned long long inc_m = my_m; unsigned int inc_c = my_c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long m2 = __shfl_up_sync(0xffffffffu, inc_m, o);
        const unsigned int c2 = __shfl_up_sync(0xffffffffu, inc_c, o);
        if (lane >= o) { inc_m += m2; inc_c += c2; }
    }
    if (tid == 0) s.pick = kSampBuckets;
    if (lane == 31) { s.sc_m[wp] = inc_m; s.sc_c[wp] = inc_c; }
    __syncthreads();
    unsigned long long off_m = 0; unsigned int off_c = 0;
#pragma unroll 8
    for (int k = 0; k < wp; ++k) { off_m += s.sc_m[k]; off_c += s.sc_c[k]; }
    inc_m += off_m; inc_c += off_c;
    if (b >= 0 && my_c > 0 && cum + inc_m >= target) atomicMin(&s.pick, tid);
    if (tid == kSampThreads - 1) { s.tot_m = inc_m; s.tot_c = inc_c; }
    __syncthreads();
    const int pick = s.pick;
    if (pick == kSampBuckets) {
        cum += s.tot_m; cnt += s.tot_c;
        __syncthreads();
        return -1;
    }
    if (tid == pick) { s.pk_above_m = inc_m - my_m; s.pk_above_c = inc_c - my_c; s.pk_m = my_m; s.pk_c = my_c; }
    __syncthreads();
    cum += s.pk_above_m; cnt += s.pk_above_c;
    bucket_mass = s.pk_m; bucket_cnt = s.pk_c;
    __syncthreads();
    return top - pick;
}

// A thread's share of the level-0 histogram: kL0PerThread consecutive buckets in descending order (k = 0 is
// the highest), with the mass and count of everything above them.
struct L0Regs {
    unsigned long long m[kL0PerThread]; unsigned int c[kL0PerThread];
    unsigned long long exc_m; unsigned int exc_c;
};

// Loads this thread's share of the slot's level-0 histogram and clears it for the next step.
__device__ __forceinline__ void l0_load(unsigned long long* gm, unsigned int* gc, L0Regs& r) {
    static_assert(kL0PerThread == 8, "vector loads below assume 8 buckets per thread");
    const int tid = threadIdx.x;
    const int base = kL0Buckets - kL0PerThread * (tid + 1);     // this thread's lowest bucket
    ulonglong2 mm[4]; uint4 cc[2];
#pragma unroll
    for (int j = 0; j < 4; ++j) mm[j] = __ldcg(reinterpret_cast<const ulonglong2*>(gm + base) + j);
#pragma unroll
    for (int j = 0; j < 2; ++j) cc[j] = __ldcg(reinterpret_cast<const uint4*>(gc + base) + j);
#pragma unroll
    for (int j = 0; j < 4; ++j) { r.m[7 - 2 * j] = mm[j].x; r.m[6 - 2 * j] = mm[j].y; }
    r.c[7] = cc[0].x; r.c[6] = cc[0].y; r.c[5] = cc[0].z; r.c[4] = cc[0].w;
    r.c[3] = cc[1].x; r.c[2] = cc[1].y; r.c[1] = cc[1].z; r.c[0] = cc[1].w;
#pragma unroll
    for (int j = 0; j < 4; ++j) reinterpret_cast<ulonglong2*>(gm + base)[j] = make_ulonglong2(0ull, 0ull);
#pragma unroll
    for (int j = 0; j < 2; ++j) reinterpret_cast<uint4*>(gc + base)[j] = make_uint4(0u, 0u, 0u, 0u);
}

// Block-wide exclusive prefix of the level-0 histogram in descending bucket order; totals in s.tot_m / s.tot_c.
__device__ void l0_scan(L0Regs& r, SampScratch& s) {
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    unsigned long long my_m = 0; unsigned int my_c = 0;
#pragma unroll
    for (int k = 0; k < kL0PerThread; ++k) { my_m += r.m[k]; my_c += r.c[k]; }
    unsigned long long inc_m = my_m; unsigned int inc_c = my_c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long m2 = __shfl_up_sync(0xffffffffu, inc_m, o);
        const unsigned int c2 = __shfl_up_sync(0xffffffffu, inc_c, o);
        if (lane >= o) { inc_m += m2; inc_c += c2; }
    }
    if (lane == 31) { s.sc_m[wp] = inc_m; s.sc_c[wp] = inc_c; }
    __syncthreads();
    unsigned long long off_m = 0; unsigned int off_c = 0;
#pragma unroll 8
    for (int k = 0; k < wp; ++k) { off_m += s.sc_m[k]; off_c += s.sc_c[k]; }
    inc_m += off_m; inc_c += off_c;
    r.exc_m = inc_m - my_m; r.exc_c = inc_c - my_c;
    if (tid == kSampThreads - 1) { s.tot_m = inc_m; s.tot_c = inc_c; }
    __syncthreads();
}

// First non-empty level-0 bucket, from the highest down, at which the running mass reaches target: returns its
// index (or -1 when the total stays below), the mass / count above it and its own.
__device__ int l0_query(const L0Regs& r, SampScratch& s, unsigned long long target, unsigned long long& above_m,
                        unsigned int& above_c, unsigned long long& bucket_mass, unsigned int& bucket_cnt) {
    const int tid = threadIdx.x;
    if (tid == 0) s.pick = kL0Buckets;
    __syncthreads();
    unsigned long long cum = r.exc_m; unsigned int cnt = r.exc_c;
    int found = -1;
#pragma unroll
    for (int k = 0; k < kL0PerThread; ++k) {
        if (found < 0) {
            if (r.c[k] > 0 && cum + r.m[k] >= target) found = k;
            else { cum += r.m[k]; cnt += r.c[k]; }
        }
    }
    if (found >= 0) atomicMin(&s.pick, tid * kL0PerThread + found);
    __syncthreads();
    const int pick = s.pick;
    if (pick == kL0Buckets) {
        above_m = s.tot_m; above_c = s.tot_c;
        __syncthreads();
        return -1;
    }
    if (pick / kL0PerThread == tid) {
        s.pk_above_m = cum; s.pk_above_c = cnt;
#pragma unroll
        for (int k = 0; k < kL0PerThread; ++k)
            if (k == found) { s.pk_m = r.m[k]; s.pk_c = r.c[k]; }
    }
    __syncthreads();
    above_m = s.pk_above_m; above_c = s.pk_above_c;
    bucket_mass = s.pk_m; bucket_cnt = s.pk_c;
    __syncthreads();
    return kL0Buckets - 1 - pick;
}

// Finds the element, in descending (key, then ascending id) order, at which the running mass first reaches
// `target`, inside the key range [lo, hi] of a level-0 bucket known to contain it; cum / cnt are the mass and count
// above that bucket; h1 is working space.
__device__ SelectResult select_mass(const float* w, int V, unsigned long long target, uint32_t lo, uint32_t hi,
                                    unsigned long long cum, unsigned int cnt, SampHist& h1, SampScratch& s) {
    const int tid = threadIdx.x;
    unsigned long long bm = 0; unsigned int bc = 0;
    SelectResult res;
    res.found = 0; res.qk = 0; res.ties = 0; res.r = 0; res.key = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int sh = shift_for(hi - lo);
        hist_clear(h1);
        __syncthreads();
        for (int i = tid; i < V; i += kSampThreads) {
            const uint32_t key = __float_as_uint(w[i]);
            if (key >= lo && key <= hi) hist_add(h1, (int)((key - lo) >> sh), fix_of(w[i]));
        }
        __syncthreads();
        const int top = (int)((hi - lo) >> sh);
        const int bb = top - tid;
        const int b = scan_pick(bb >= 0 ? hist_mass(h1, bb) : 0ull, bb >= 0 ? h1.cnt[bb] : 0u, top, s, target, cum, cnt, bm, bc);
        if (b < 0) break;                        // cannot happen: the parent bucket contained the crossing
        const uint32_t nlo = lo + ((uint32_t)b << sh);
        uint32_t nhi = (sh == 0) ? nlo : (nlo + ((1u << sh) - 1u));
        if (nhi > hi) nhi = hi;
        lo = nlo; hi = nhi;
        if (sh == 0) {                           // one key per bucket: done
            res.found = 1; res.key = lo; res.ties = bc; res.qk = bm / bc;
            const unsigned long long need = target > cum ? target - cum : 0;
            unsigned long long r = res.qk ? (need + res.qk - 1) / res.qk : 1;
            if (r < 1) r = 1;
            if (r > bc) r = bc;
            res.r = (unsigned int)r;
            break;
        }
    }
    res.cum_above = cum; res.cnt_above = cnt;
    return res;
}

// id of the r-th (1-based) lowest index whose weight has bit pattern `key`.  Warp w owns a contiguous block of
// ids and walks it 32 at a time (conflict-free shared-memory reads); ballots keep the order by id.
__device__ int nth_with_key(const float* w, int V, uint32_t key, unsigned int r, unsigned int* s_scan, int* s_out) {
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const int per_warp = ((V + 31) / 32 + 31) / 32 * 32;       // ids per warp, a multiple of 32
    const int b = wp * per_warp, e = min(V, b + per_warp);
    unsigned int c = 0;
    for (int i = b; i < e; i += 32) {
        const bool m = (i + lane < e) && __float_as_uint(w[i + lane]) == key;
        c += __popc(__ballot_sync(0xffffffffu, m));
    }
    if (lane == 0) s_scan[wp] = c;
    if (tid == 0) *s_out = -1;
    __syncthreads();
    unsigned int before = 0;
    for (int k = 0; k < wp; ++k) before += s_scan[k];
    if (c > 0 && r > before && r <= before + c) {              // warp-uniform
        unsigned int rr = r - before;
        for (int i = b; i < e; i += 32) {
            const bool m = (i + lane < e) && __float_as_uint(w[i + lane]) == key;
            const unsigned int bal = __ballot_sync(0xffffffffu, m);
            const unsigned int n = __popc(bal);
            if (rr <= n) {
                if (lane == 0) *s_out = i + (int)__fns(bal, 0, (int)rr);
                break;
            }
            rr -= n;
        }
    }
    __syncthreads();
    const int out = *s_out;
    __syncthreads();
    return out;
}

// Exact answer inside one level-0 bucket when it holds at most kSampCand elements: gather them, order them by
// (weight descending, id ascending) by rank counting, running mass by a block scan.  Returns the position of the
// crossing element in that order (or -1), its id, and the mass / count up to and including it.
constexpr int kSampCand = 1024;
struct CandScratch {
    uint32_t key[kSampCand], skey[kSampCand];
    int id[kSampCand], sid[kSampCand];
    unsigned long long warp_m[32];
    int n, pick;
};
__device__ int cand_solve(const float* w, int V, uint32_t lo, uint32_t hi, unsigned int n_expect, unsigned long long need,
                          CandScratch& cs, int& id_out, unsigned long long& mass_incl, unsigned int& cnt_incl) {
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    if (tid == 0) { cs.n = 0; cs.pick = kSampCand; }
    __syncthreads();
    auto take = [&](uint32_t k, int i) {
        if (k >= lo && k <= hi) {
            const int p = atomicAdd(&cs.n, 1);
            if (p < kSampCand) { cs.key[p] = k; cs.id[p] = i; }
        }
    };
    // 16 bytes per shared-memory load (the list's order does not matter: the candidates are ranked below)
    const int V4 = V & ~3;
    for (int i = tid * 4; i < V4; i += kSampThreads * 4) {
        const uint4 k = *reinterpret_cast<const uint4*>(w + i);
        take(k.x, i); take(k.y, i + 1); take(k.z, i + 2); take(k.w, i + 3);
    }
    for (int i = V4 + tid; i < V; i += kSampThreads) take(__float_as_uint(w[i]), i);
    __syncthreads();
    const int n = min(cs.n, kSampCand);
    (void)n_expect;
    uint32_t mk = 0; int mi = 0;
    if (tid < n) {
        mk = cs.key[tid]; mi = cs.id[tid];
        int rank = 0;
#pragma unroll 8
        for (int j = 0; j < n; ++j) {
            const uint32_t kj = cs.key[j];
            rank += (kj > mk) || (kj == mk && cs.id[j] < mi);
        }
        cs.skey[rank] = mk; cs.sid[rank] = mi;
    }
    __syncthreads();
    unsigned long long q = tid < n ? fix_of(__uint_as_float(cs.skey[tid])) : 0ull;
    unsigned long long inc = q;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long m2 = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += m2;
    }
    if (lane == 31) cs.warp_m[wp] = inc;
    __syncthreads();
    unsigned long long off = 0;
#pragma unroll 8
    for (int k = 0; k < wp; ++k) off += cs.warp_m[k];
    inc += off;
    if (tid < n && inc >= need) atomicMin(&cs.pick, tid);
    __syncthreads();
    const int pick = cs.pick;
    __shared__ unsigned long long s_mass;
    if (pick < kSampCand && tid == pick) s_mass = inc;
    __syncthreads();
    if (pick >= kSampCand) return -1;
    id_out = cs.sid[pick];
    mass_incl = s_mass;
    cnt_incl = (unsigned int)pick + 1u;
    __syncthreads();
    return pick;
}

// Where the descending running mass first reaches `target`: through the candidate solver when the level-0
// bucket is small enough (the usual case), else through the histogram refinement.
struct Loc { int found, have_id, id; unsigned long long mass_incl; unsigned int cnt_incl; uint32_t key; unsigned int r; };
__device__ Loc locate(const float* w, int V, unsigned long long target, const L0Regs& l0, SampHist& h1, SampScratch& sc,
                      CandScratch& cs) {
    Loc L; L.found = 0; L.have_id = 0; L.id = -1; L.key = 0; L.r = 0;
    unsigned long long cum = 0, bm = 0; unsigned int cnt = 0, bc = 0;
    const int b = l0_query(l0, sc, target, cum, cnt, bm, bc);
    if (b < 0) { L.mass_incl = cum; L.cnt_incl = cnt; return L; }
    uint32_t lo, hi;
    l0_range(b, lo, hi);
    if (bc <= (unsigned int)kSampCand) {
        unsigned long long m = 0; unsigned int c = 0; int id = -1;
        const int pick = cand_solve(w, V, lo, hi, bc, target > cum ? target - cum : 0ull, cs, id, m, c);
        if (pick >= 0) { L.found = 1; L.have_id = 1; L.id = id; L.mass_incl = cum + m; L.cnt_incl = cnt + c; return L; }
    }
    const SelectResult r = select_mass(w, V, target, lo, hi, cum, cnt, h1, sc);
    L.found = r.found; L.key = r.key; L.r = r.r;
    L.mass_incl = r.found ? r.cum_above + (unsigned long long)r.r * r.qk : r.cum_above;
    L.cnt_incl = r.found ? r.cnt_above + r.r : r.cnt_above;
    return L;
}

constexpr int kSampPartThreads = 256;

__device__ __forceinline__ float penalised(const SampleArgs& a, const float* lg, const uint32_t* seen, int i) {
    float s = lg[i];
    if (a.penalty != 1.0f && ((seen[i >> 5] >> (i & 31)) & 1u)) s = s > 0.f ? s / a.penalty : s * a.penalty;
    return s;
}
__device__ __forceinline__ void first_max(float& bv, int& bi, float v2, int i2) {
    if (v2 > bv || (v2 == bv && i2 < bi)) { bv = v2; bi = i2; }
}

// per-block first maximum of the penalised scores: grid (bps, n_slots)
__global__ void __launch_bounds__(kSampPartThreads) k_samp_max(const SampleArgs a) {
    __shared__ float r_val[kSampPartThreads / 32];
    __shared__ int r_idx[kSampPartThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    SLLM_TL(300);
    const int slot = blockIdx.y, tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const int per = (a.V + a.bps - 1) / a.bps, b0 = blockIdx.x * per, b1 = min(a.V, b0 + per);
    const float* lg = a.logits + (size_t)slot * a.V;
    const uint32_t* seen = a.st.seen + (size_t)slot * (a.V / 32);
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = b0 + tid; i < b1; i += kSampPartThreads) {
        const float s = penalised(a, lg, seen, i);
        if (s > bv) { bv = s; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) first_max(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) { r_val[wp] = bv; r_idx[wp] = bi; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < kSampPartThreads / 32; ++w) first_max(bv, bi, r_val[w], r_idx[w]);
        a.g_pmax_val[(size_t)slot * a.bps + blockIdx.x] = bv;
        a.g_pmax_idx[(size_t)slot * a.bps + blockIdx.x] = bi;
    }
}

// the slot's maximum from the per-block maxima (every thread of the block calls it; needs one __syncthreads pair)
__device__ __forceinline__ void slot_max(const SampleArgs& a, int slot, float* s_val, int* s_idx, float& mx, int& arg) {
    const int tid = threadIdx.x;
    if (tid < 32) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int b = tid; b < a.bps; b += 32)
            first_max(bv, bi, __ldcg(a.g_pmax_val + (size_t)slot * a.bps + b), __ldcg(a.g_pmax_idx + (size_t)slot * a.bps + b));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) first_max(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (tid == 0) { *s_val = bv; *s_idx = bi; }
    }
    __syncthreads();
    mx = *s_val; arg = *s_idx;
}

// weights and level-0 histogram: grid (bps, n_slots)
__global__ void __launch_bounds__(kSampPartThreads) k_samp_hist(const SampleArgs a) {
    __shared__ float s_val; __shared__ int s_idx;
    pdl_launch_dependents();
    pdl_wait();
    SLLM_TL(310);
    const int slot = blockIdx.y, tid = threadIdx.x;
    const int per = (a.V + a.bps - 1) / a.bps, b0 = blockIdx.x * per, b1 = min(a.V, b0 + per);
    const float* lg = a.logits + (size_t)slot * a.V;
    const uint32_t* seen = a.st.seen + (size_t)slot * (a.V / 32);
    // the thread's first element is requested before the maximum's reduction (with one block row per SM it is
    // the only one), so the two round trips overlap
    const int i0 = b0 + tid;
    const float raw0 = i0 < b1 ? lg[i0] : 0.f;
    const uint32_t word0 = i0 < b1 ? seen[i0 >> 5] : 0u;
    if (a.st.finished[slot]) return;
    float mx; int arg;
    slot_max(a, slot, &s_val, &s_idx, mx, arg);
    if (!isfinite(mx)) return;
    float* w = a.g_w + (size_t)slot * a.V;
    unsigned long long* gm = a.g_mass + (size_t)slot * kL0Buckets;
    unsigned int* gc = a.g_cnt + (size_t)slot * kL0Buckets;
    for (int i = i0; i < b1; i += kSampPartThreads) {
        float sv = i == i0 ? raw0 : lg[i];
        const uint32_t word = i == i0 ? word0 : seen[i >> 5];
        if (a.penalty != 1.0f && ((word >> (i & 31)) & 1u)) sv = sv > 0.f ? sv / a.penalty : sv * a.penalty;
        const float e = expf((sv - mx) / a.temperature);
        w[i] = e;
        const int b = l0_bucket(__float_as_uint(e));
        atomicAdd(gm + b, fix_of(e));              // results unused: reductions performed in L2
        atomicAdd(gc + b, 1u);
    }
}

// one block per slot: top-p cut, draw, append, stop rules, inputs of the next decode pass
__global__ void __launch_bounds__(kSampThreads) k_samp_pick(const SampleArgs a) {
    extern __shared__ __align__(16) float w[];                 // [V] weights
    __shared__ SampHist h1;
    __shared__ SampScratch sc;
    __shared__ CandScratch cs;
    __shared__ unsigned int s_scan[32];
    __shared__ int s_out;
    __shared__ float s_val; __shared__ int s_idx;

    const int slot = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const int V = a.V;
    PS_TL_INIT(16);
    pdl_launch_dependents();
    pdl_wait();

    PS_TL(320);
    // Everything the sampling path reads from global memory is requested up front, ahead of the maximum's reduction:
    // the first trip of the weights and this thread's share of the level-0 histogram (which is cleared for the
    // next step; a finished slot's histogram is empty and its weights are not used).
    const bool sampling = a.temperature > 0.0f;
    unsigned long long* gm = a.g_mass + (size_t)slot * kL0Buckets;
    unsigned int* gc = a.g_cnt + (size_t)slot * kL0Buckets;
    const float* gw = a.g_w + (size_t)slot * V;
    float pv[4]; int pi[4];                                    // warp 0: the per-block maxima (bps <= 128)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int b = tid + 32 * k;
        const bool in = tid < 32 && b < a.bps;
        pv[k] = in ? __ldcg(a.g_pmax_val + (size_t)slot * a.bps + b) : -INFINITY;
        pi[k] = in ? __ldcg(a.g_pmax_idx + (size_t)slot * a.bps + b) : 0x7fffffff;
    }
    int n_tok = a.st.n_tok[slot];
    const int fin = a.st.finished[slot];
    double u = 0.0;
    if (sampling && a.draws) u = a.draws[(size_t)slot * a.draws_stride + min(a.st.draw_idx[slot], a.draws_stride - 1)];
    L0Regs l0;
    if (sampling) {
        l0_load(gm, gc, l0);
        for (int base = 0; base < V; base += kSampThreads * 4 * 8) {          // 8 independent 16-byte loads per thread and trip
            float4 t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = base + (j * kSampThreads + tid) * 4;
                t[j] = i < V ? __ldcg(reinterpret_cast<const float4*>(gw + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = base + (j * kSampThreads + tid) * 4;
                if (i < V) *reinterpret_cast<float4*>(w + i) = t[j];
            }
        }
    }
    PS_TL(3201);
    // the slot's maximum (first index among equals) from the per-block maxima
    if (tid < 32) {
        float bv = pv[0]; int bi = pi[0];
#pragma unroll
        for (int k = 1; k < 4; ++k) first_max(bv, bi, pv[k], pi[k]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) first_max(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (tid == 0) { s_val = bv; s_idx = bi; }
    }
    __syncthreads();
    PS_TL(3202);
    const float mx = s_val; const int arg = s_idx;
    int token = -1;
    if (!fin) {
        if (!isfinite(mx)) {
            if (tid == 0) a.st.finished[slot] = 3;
        } else if (!sampling) {
            token = arg;
        } else {
            l0_scan(l0, sc);                                   // ends with a block barrier: w is complete too
            const unsigned long long total = sc.tot_m;
            PS_TL(322);
            // ---- top-p: first prefix whose mass reaches top_p of the total -----------------------
            unsigned long long t1 = (unsigned long long)ceil((double)a.top_p * (double)total);
            if (t1 > total) t1 = total + 1;                    // unreachable: everything is kept
            const Loc cut = locate(w, V, t1, l0, h1, sc, cs);
            const unsigned long long kept_mass = cut.mass_incl;
            const unsigned int kept = cut.cnt_incl;
            PS_TL(323);
            // ---- the draw -------------------------------------------------------------------------
            unsigned long long t2 = (unsigned long long)ceil(u * (double)kept_mass);
            if (t2 > kept_mass) t2 = kept_mass;
            const Loc hit = locate(w, V, t2, l0, h1, sc, cs);
            PS_TL(324);
            const Loc& use = (hit.found && hit.cnt_incl <= kept) ? hit : cut;    // else: the last kept candidate
            if (use.found) {
                token = use.have_id ? use.id : nth_with_key(w, V, use.key, use.r, s_scan, &s_out);
            } else {                                                             // last of everything: highest id of the smallest weight
                uint32_t kmin = 0xffffffffu;
                for (int i = tid; i < V; i += kSampThreads) kmin = min(kmin, __float_as_uint(w[i]));
                kmin = __reduce_min_sync(0xffffffffu, kmin);
                if (lane == 0) s_scan[wp] = kmin;
                __syncthreads();
                for (int i = 0; i < 32; ++i) kmin = min(kmin, s_scan[i]);
                __syncthreads();
                unsigned int c = 0;
                for (int i = tid; i < V; i += kSampThreads) c += (__float_as_uint(w[i]) == kmin);
                c = __reduce_add_sync(0xffffffffu, c);
                if (lane == 0) s_scan[wp] = c;
                __syncthreads();
                unsigned int t = 0;
                for (int i = 0; i < 32; ++i) t += s_scan[i];
                __syncthreads();
                token = nth_with_key(w, V, kmin, t, s_scan, &s_out);
            }
            PS_TL(325);
            if (tid == 0 && (!a.seeded || kept >= 2)) a.st.draw_idx[slot] += 1;
        }
    }

    // ---- append, stop rules, next pass inputs ------------------------------------------------------
    if (tid == 0) {
        int f = a.st.finished[slot];
        if (!f && token >= 0) {
            a.st.tokens[(size_t)slot * a.st.tok_cap + n_tok] = (uint32_t)token;
            n_tok += 1;
            a.st.n_tok[slot] = n_tok;
            atomicOr(&a.st.seen[(size_t)slot * (V / 32) + (token >> 5)], 1u << (token & 31));
            if ((uint32_t)token == a.eos || (long long)token == a.stop_token) f = 1;
            else if (n_tok > a.ctx) f = 2;
            a.st.finished[slot] = f;
        }
        // the decode step that follows feeds the last token at position n_tok-1; finished slots
        // repeat their last position (idempotent) so the launch shape stays fixed
        const int p = min(n_tok - 1, a.ctx - 1);
        a.next_tok_id[slot] = a.st.tokens[(size_t)slot * a.st.tok_cap + p];
        a.next_tok_pos[slot] = p;
        a.next_tok_slot[slot] = slot;
    }
    PS_TL(321);
}

}  // namespace sllm
