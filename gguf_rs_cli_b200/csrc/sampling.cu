// Sampling on the device, a cluster of up to eight CTAs per sequence, in the order of the reference's
// sampler (src/sampler.rs:35-79): repetition penalty on recently emitted tokens;
// temperature <= 0 takes the largest logit; else logits / temperature, the top_k
// largest survive, softmax over them, top_p keeps the smallest set of the most
// probable whose mass reaches it, and one uniform picks a survivor.
//
// Differences from the reference, on purpose: the vocabulary is never sorted.  The k-th
// largest value is found as a threshold over the ordered bit patterns of the floats (four
// passes of eight bits with a histogram each), ties at a threshold go to the lower indices,
// and the cumulative walk runs over the survivors in index order (the same distribution).
// With a top_k of up to 1,024 the survivors are gathered into shared memory, and what
// follows (top_p in descending order, the walk) runs on that list.  Without top_k the walk
// goes over the whole vocabulary, each warp with a contiguous piece of it, and the edge of the
// nucleus is found like the k-th largest value, with masses in the histogram (in fixed point,
// so that their sums do not depend on the order).  A top_k above 1,024 finds its thresholds
// by bisection, one bit a pass.
// The uniform comes from a counter-based generator per sequence:
// top 24 bits of splitmix64(seed + (n+1) * golden), n = number of tokens sampled so
// far for that sequence; the reference's single global LCG divides a 31-bit value by
// 2^32, so its draws never exceed one half (src/sampler.rs:7-12).
//
// Per-sequence state lives in the cache's fixed-size state area, indexed by slot:
// recent[slot][64] (ring of emitted tokens, src/main.rs:302-303) and count[slot].
#include <math.h>

#include "common.cuh"

constexpr int SM_THREADS = 1024;
constexpr int SM_WARPS = SM_THREADS / 32;
constexpr int SM_RECENT = 64;
constexpr int SM_LIST = 1024;            // survivors of top_k that are worked on in shared memory

__device__ __forceinline__ unsigned ordered_key(float z) {
    unsigned u = __float_as_uint(z);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Block-wide sum that every thread receives.
template <typename T> __device__ T block_sum(T v, T* scratch) {
    __syncthreads();
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    T r = 0;
    for (int w = 0; w < SM_THREADS / 32; ++w) r += scratch[w];
    return r;
}

// Exclusive prefix over threads (in thread order) of v; also returns the total.
__device__ int block_exclusive_scan(int v, int* scratch, int* total) {
    __syncthreads();
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    int base = 0, tot = 0;
    for (int w = 0; w < SM_THREADS / 32; ++w) {
        if (w < warp) base += scratch[w];
        tot += scratch[w];
    }
    *total = tot;
    return base + inc - v;
}

__device__ float block_exclusive_scan_f(float v, float* scratch, float* total) {
    __syncthreads();
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float inc = v;
    for (int o = 1; o < 32; o <<= 1) {
        float n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    float base = 0.f, tot = 0.f;
    for (int w = 0; w < SM_THREADS / 32; ++w) {
        if (w < warp) base += scratch[w];
        tot += scratch[w];
    }
    *total = tot;
    return base + inc - v;
}

// Thresholds by bisection over the whole vocabulary, every thread with a contiguous range of it: any
// combination of top_k and top_p, one pass over the logits per bit.
__device__ int sample_by_bisection(const float* __restrict__ z, int V, float temperature, int top_k, float top_p, float bv,
                                   int bi, float u, float* fs, int* is, int* best_i) {
    const int tid = threadIdx.x;
    float zmax = bv / temperature;
    // contiguous index range of this thread, for everything that depends on index order
    int chunk = (V + SM_THREADS - 1) / SM_THREADS;
    int c0 = min(V, tid * chunk), c1 = min(V, c0 + chunk);

    // 3. top_k: threshold key tk = the k-th largest; `k_eq` of the elements equal to it survive
    unsigned tk = 0;
    int k_eq = 0x7fffffff;
    bool use_k = top_k > 0 && top_k < V;
    if (use_k) {
        for (int bit = 31; bit >= 0; --bit) {
            unsigned cand = tk | (1u << bit);
            int c = 0;
            for (int i = tid; i < V; i += SM_THREADS) c += ordered_key(z[i] / temperature) >= cand;
            if (block_sum<int>(c, is) >= top_k) tk = cand;
        }
        int c = 0;
        for (int i = tid; i < V; i += SM_THREADS) c += ordered_key(z[i] / temperature) > tk;
        k_eq = top_k - block_sum<int>(c, is);
    }
    // rank, in index order, of this thread's first element among those equal to tk
    int eqk_before = 0;
    if (use_k) {
        int c = 0, tot;
        for (int i = c0; i < c1; ++i) c += ordered_key(z[i] / temperature) == tk;
        eqk_before = block_exclusive_scan(c, is, &tot);
    }
    // survivors of top_k: key > tk, or key == tk with rank < k_eq
    // 4. their mass
    float mass = 0.f;
    {
        int r = eqk_before;
        for (int i = c0; i < c1; ++i) {
            float zi = z[i] / temperature;
            unsigned key = ordered_key(zi);
            bool s = !use_k || key > tk || (key == tk && r < k_eq);
            if (use_k && key == tk) ++r;
            if (s) mass += expf(zi - zmax);
        }
    }
    float Z = block_sum<float>(mass, fs);

    // 5. top_p: threshold key tp = lowest value still inside the nucleus; p_eq of the equal ones survive
    bool use_p = top_p < 1.0f;
    unsigned tp = 0;
    int p_eq = 0x7fffffff;
    if (use_p) {
        float goal = top_p * Z;
        for (int bit = 31; bit >= 0; --bit) {
            unsigned cand = tp | (1u << bit);
            float msum = 0.f;
            int r = eqk_before;
            for (int i = c0; i < c1; ++i) {
                float zi = z[i] / temperature;
                unsigned key = ordered_key(zi);
                bool s = !use_k || key > tk || (key == tk && r < k_eq);
                if (use_k && key == tk) ++r;
                if (s && key >= cand) msum += expf(zi - zmax);
            }
            if (block_sum<float>(msum, fs) >= goal) tp = cand;
        }
        float mgt = 0.f, e_eq = 0.f;
        int r = eqk_before;
        for (int i = c0; i < c1; ++i) {
            float zi = z[i] / temperature;
            unsigned key = ordered_key(zi);
            bool s = !use_k || key > tk || (key == tk && r < k_eq);
            if (use_k && key == tk) ++r;
            if (s && key > tp) mgt += expf(zi - zmax);
            if (s && key == tp) e_eq = expf(zi - zmax);
        }
        mgt = block_sum<float>(mgt, fs);
        // every element equal to tp has the same weight; any thread that saw one knows it
        float e_all = e_eq;
        for (int o = 16; o > 0; o >>= 1) e_all = fmaxf(e_all, __shfl_xor_sync(0xffffffffu, e_all, o));
        __syncthreads();
        if ((tid & 31) == 0) fs[tid >> 5] = e_all;
        __syncthreads();
        e_all = 0.f;
        for (int w = 0; w < SM_THREADS / 32; ++w) e_all = fmaxf(e_all, fs[w]);
        __syncthreads();
        // the smallest count c with mgt + c * e >= goal, accumulated as the reference does
        int c = 1;
        float cum = mgt + e_all;
        while (cum < goal && c < V) { cum += e_all; ++c; }
        p_eq = c;
    }
    // rank among elements equal to tp (same ranks as for tk when the thresholds coincide)
    int eqp_before = 0;
    if (use_p) {
        int c = 0, tot;
        for (int i = c0; i < c1; ++i) c += ordered_key(z[i] / temperature) == tp;
        eqp_before = block_exclusive_scan(c, is, &tot);
    }

    // 6. mass of the final survivors, in index order, and the walk
    float mine = 0.f;
    {
        int rk = eqk_before, rp = eqp_before;
        for (int i = c0; i < c1; ++i) {
            float zi = z[i] / temperature;
            unsigned key = ordered_key(zi);
            bool s = !use_k || key > tk || (key == tk && rk < k_eq);
            if (use_p) s = s && (key > tp || (key == tp && rp < p_eq));
            if (use_k && key == tk) ++rk;
            if (use_p && key == tp) ++rp;
            if (s) mine += expf(zi - zmax);
        }
    }
    float Z2;
    float before = block_exclusive_scan_f(mine, fs, &Z2);
    float target = u * Z2;
    __syncthreads();
    // the last survivor overall is the fallback (src/sampler.rs:78); first the walk
    int last_surv = -1, hit = -1;
    {
        int rk = eqk_before, rp = eqp_before;
        float cum = before;
        for (int i = c0; i < c1; ++i) {
            float zi = z[i] / temperature;
            unsigned key = ordered_key(zi);
            bool s = !use_k || key > tk || (key == tk && rk < k_eq);
            if (use_p) s = s && (key > tp || (key == tp && rp < p_eq));
            if (use_k && key == tk) ++rk;
            if (use_p && key == tp) ++rp;
            if (s) {
                cum += expf(zi - zmax);
                last_surv = i;
                if (hit < 0 && target < cum) hit = i;
            }
        }
    }
    // lowest hit over the block; else the highest survivor
    int h = hit < 0 ? 0x7fffffff : hit;
    for (int o = 16; o > 0; o >>= 1) h = min(h, __shfl_xor_sync(0xffffffffu, h, o));
    int ls = last_surv;
    for (int o = 16; o > 0; o >>= 1) ls = max(ls, __shfl_xor_sync(0xffffffffu, ls, o));
    __syncthreads();
    if ((tid & 31) == 0) { is[tid >> 5] = h; best_i[tid >> 5] = ls; }
    __syncthreads();
    h = 0x7fffffff; ls = -1;
    for (int w = 0; w < SM_THREADS / 32; ++w) { h = min(h, is[w]); ls = max(ls, best_i[w]); }
    return h != 0x7fffffff ? h : (ls >= 0 ? ls : bi);
}

// Calls f(index, value) for every logit of the row, the block's threads reading neighbouring elements (four
// each where the row allows 16-byte loads).  The loads of a round (four a thread) are issued before any of
// them is used: a pass over the row costs round trips to L2, not arithmetic.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* z, int V, F f) {
    const int tid = threadIdx.x;
    if ((reinterpret_cast<uintptr_t>(z) & 15) == 0) {
        const float4* z4 = reinterpret_cast<const float4*>(z);
        const int n4 = V >> 2;
        for (int j0 = 0; j0 < n4; j0 += 4 * SM_THREADS) {
            float4 v[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int j = j0 + r * SM_THREADS + tid;
                v[r] = j < n4 ? z4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int j = j0 + r * SM_THREADS + tid;
                if (j < n4) {
                    f(4 * j, v[r].x);
                    f(4 * j + 1, v[r].y);
                    f(4 * j + 2, v[r].z);
                    f(4 * j + 3, v[r].w);
                }
            }
        }
        for (int i = 4 * n4 + tid; i < V; i += SM_THREADS) f(i, z[i]);
    } else {
#pragma unroll 4
        for (int i = tid; i < V; i += SM_THREADS) f(i, z[i]);
    }
}

// The same with every thread of the block making the same number of calls (`valid` false beyond the row), for
// callers whose f talks to the other lanes of its warp.
template <typename F>
__device__ __forceinline__ void for_each_logit_in_step(const float* z, int V, F f) {
    const int tid = threadIdx.x;
    if ((reinterpret_cast<uintptr_t>(z) & 15) == 0) {
        const float4* z4 = reinterpret_cast<const float4*>(z);
        const int n4 = V >> 2;
        for (int j0 = 0; j0 < n4; j0 += 4 * SM_THREADS) {
            float4 v[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int j = j0 + r * SM_THREADS + tid;
                v[r] = j < n4 ? z4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const bool valid = j0 + r * SM_THREADS + tid < n4;
                f(v[r].x, valid);
                f(v[r].y, valid);
                f(v[r].z, valid);
                f(v[r].w, valid);
            }
        }
        const int i = 4 * n4 + tid;                         // the up to three elements left over
        f(i < V ? z[i] : 0.f, i < V);
    } else {
        for (int i0 = 0; i0 < V; i0 += 4 * SM_THREADS) {
            float v[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) v[r] = i0 + r * SM_THREADS + tid < V ? z[i0 + r * SM_THREADS + tid] : 0.f;
#pragma unroll
            for (int r = 0; r < 4; ++r) f(v[r], i0 + r * SM_THREADS + tid < V);
        }
    }
}

// A warp's piece [seg0, seg1) of the row, 512 elements a round: the sixteen loads of a round are issued
// together, then f(index, value, inside) runs sixteen times on 32 neighbouring elements each, in index order
// (every lane calls it, `inside` false beyond the piece).  f returns false to stop.
template <typename F>
__device__ __forceinline__ void for_each_in_piece(const float* z, int seg0, int seg1, int lane, F f) {
    constexpr int R = 16;
    bool go = true;
    for (int base = seg0; base < seg1 && go; base += 32 * R) {
        float v[R];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int i = base + 32 * q + lane;
            v[q] = i < seg1 ? z[i] : 0.f;
        }
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int i = base + 32 * q + lane;
            if (go && base + 32 * q < seg1) go = f(i, v[q], i < seg1);
        }
    }
}

// exp(d), d <= 0, in 64-bit fixed point with 40 binary places: sums of these do not depend on their order.
__device__ __forceinline__ unsigned long long fixed_mass(float d) { return __float2ull_rn(expf(d) * 1099511627776.0f); }

// Inclusive sum over the lanes of a warp, in lane order.
__device__ __forceinline__ float warp_inclusive(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
    }
    return v;
}

// ------------------------------------------------------ a cluster of CTAs per sequence
// The CTAs of a cluster share one row: each takes a contiguous part of it (a multiple of 128 logits), and what
// they have to tell each other (largest values, histograms, counts, masses) they read from each other's shared
// memory after a cluster barrier.  A cluster of one CTA is the plain case.
constexpr int SM_MAX_CLUSTER = 8;

__device__ __forceinline__ unsigned cl_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned cl_size() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// Every thread of every CTA of the cluster executes this; what was written before it, to shared or to global
// memory, is visible to all of them after it.
__device__ __forceinline__ void cl_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address that CTA `rank` of the cluster has for what this CTA calls p (a __shared__ variable).
__device__ __forceinline__ unsigned cl_addr(const void* p, unsigned rank) {
    unsigned a = unsigned(__cvta_generic_to_shared(p)), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ int cl_load(const int* p, unsigned rank) {
    int v;
    asm volatile("ld.shared::cluster.b32 %0, [%1];" : "=r"(v) : "r"(cl_addr(p, rank)) : "memory");
    return v;
}
__device__ __forceinline__ float cl_load(const float* p, unsigned rank) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cl_addr(p, rank)) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long cl_load(const unsigned long long* p, unsigned rank) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.b64 %0, [%1];" : "=l"(v) : "r"(cl_addr(p, rank)) : "memory");
    return v;
}
__device__ __forceinline__ void cl_store(int* p, unsigned rank, int v) {
    asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(cl_addr(p, rank)), "r"(v) : "memory");
}
__device__ __forceinline__ void cl_store(float* p, unsigned rank, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cl_addr(p, rank)), "f"(v) : "memory");
}

// One warp over a histogram of 256 bins: walking down from bin 255 with `above` as the sum so far, the first bin
// with above + h[bin] >= goal (bin 0 if none), and the sum of the bins above it (on top of the `above` given).
// Every lane takes eight bins; the lanes' sums are added up from the top lane down.
template <typename T>
__device__ __forceinline__ void pick_bin(const T* h, T goal, int lane, int& bin, T& above) {
    T c[8], s = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { c[j] = h[8 * lane + j]; s += c[j]; }
    T suf = s;                                             // this lane's bins and all bins above them
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T n = __shfl_down_sync(0xffffffffu, suf, o);
        if (lane + o < 32) suf += n;
    }
    T ab = above + (suf - s);                              // everything above this lane's bins
    const unsigned mask = __ballot_sync(0xffffffffu, ab + s >= goal);
    const int src = mask ? 31 - __clz(mask) : 0;           // the highest lane in whose bins the goal is reached
    int b = 0;
    if (mask) {
        b = 8 * lane;
#pragma unroll
        for (int j = 7; j >= 0; --j) {
            if (ab + c[j] >= goal) { b = 8 * lane + j; break; }
            ab += c[j];
        }
    } else {
        ab = above + suf - c[0];                           // (lane 0) all bins but the lowest
    }
    bin = __shfl_sync(0xffffffffu, b, src);
    above = __shfl_sync(0xffffffffu, ab, src);
}

// Which of n masses (in order, after `before`) holds the target; `before` becomes the mass in front of it.
__device__ __forceinline__ int holder_of(const float* m, int n, float target, float& before) {
    int sel = -1;
    float runsum = before;
    for (int w = 0; w < n; ++w) {
        if (sel < 0 && target < runsum + m[w]) { sel = w; before = runsum; }
        runsum += m[w];
    }
    return sel;
}

__global__ void __launch_bounds__(SM_THREADS) sample_kernel(float* __restrict__ logits, long long ld, int V,
                                                            const int* __restrict__ slots,
                                                            const long long* __restrict__ seeds, float temperature,
                                                            int top_k, float top_p, float rep_penalty,
                                                            int* __restrict__ recent, int* __restrict__ count,
                                                            int* __restrict__ out) {
    __shared__ float fs[32];
    __shared__ int is[32];
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    __shared__ float am_v;                                 // this CTA's largest value and its index, for the others
    __shared__ int am_i;
    __shared__ int cnt_s, tot_gt, tot_eq;                  // counts of this CTA, for the others
    __shared__ int chosen;
    __shared__ int hist[2][256], hist_all[256];
    __shared__ unsigned sel_prefix;
    __shared__ int sel_need;
    __shared__ int gt_s[SM_WARPS], eq_s[SM_WARPS];
    __shared__ int list_idx[SM_LIST];
    __shared__ float list_z[SM_LIST], list_e[SM_LIST], sorted_e[SM_LIST];
    __shared__ short sorted_pos[SM_LIST];
    __shared__ int cut_s;
    __shared__ unsigned long long mh[2][256], mh_all[256];
    __shared__ unsigned long long sel_above, sel_goal;
    __shared__ float all_m[SM_MAX_CLUSTER * SM_WARPS];     // every warp's mass, of every CTA
    __shared__ int all_last[SM_MAX_CLUSTER * SM_WARPS];
    gb_grid_launch_dependents();
    gb_grid_wait();
    const unsigned rank = cl_rank(), C = cl_size();
    const int row = blockIdx.x / int(C), tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slot = slots[row];
    if (slot < 0) {                                        // the whole cluster leaves
        if (rank == 0 && tid == 0) out[row] = 0;
        return;
    }
    float* zrow = logits + size_t(row) * ld;
    // this CTA's part [lo, hi) of the row; z[i] is logit lo + i
    const int part = ((V + int(C) - 1) / int(C) + 127) / 128 * 128;
    const int lo = min(V, int(rank) * part), hi = min(V, lo + part), n = hi - lo;
    float* z = zrow + lo;
    const int n_before = count[slot];

    // 1. repetition penalty, once per occurrence in the ring (src/sampler.rs:23-30), on the tokens of this part
    if (rep_penalty != 1.0f && tid == 0) {
        const int m = min(n_before, SM_RECENT);
        for (int i = 0; i < m; ++i) {
            const int tok = recent[size_t(slot) * SM_RECENT + i];
            if (tok >= lo && tok < hi) zrow[tok] = zrow[tok] > 0.f ? zrow[tok] / rep_penalty : zrow[tok] * rep_penalty;
        }
    }
    __syncthreads();

    // 2. the largest logit and its lowest index; with a temperature the row becomes logits / temperature on
    // the way (src/sampler.rs:41), which every later pass reads
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if (temperature > 0.f && (reinterpret_cast<uintptr_t>(z) & 15) == 0) {
        float4* z4 = reinterpret_cast<float4*>(z);
        const int n4 = n >> 2;
        for (int j0 = 0; j0 < n4; j0 += 4 * SM_THREADS) {
            float4 v[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int j = j0 + r * SM_THREADS + tid;
                v[r] = j < n4 ? z4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int j = j0 + r * SM_THREADS + tid;
                if (j < n4) {
                    const float e[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (e[q] > bv || (e[q] == bv && lo + 4 * j + q < bi)) { bv = e[q]; bi = lo + 4 * j + q; }
                    z4[j] = make_float4(e[0] / temperature, e[1] / temperature, e[2] / temperature, e[3] / temperature);
                }
            }
        }
        for (int i = 4 * n4 + tid; i < n; i += SM_THREADS) {
            const float v = z[i];
            if (v > bv || (v == bv && lo + i < bi)) { bv = v; bi = lo + i; }
            z[i] = v / temperature;
        }
    } else {
        for_each_logit(z, n, [&](int i, float v) {
            if (v > bv || (v == bv && lo + i < bi)) { bv = v; bi = lo + i; }
            if (temperature > 0.f) z[i] = v / temperature;
        });
    }
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (tid == 0) {
        bv = best_v[0]; bi = best_i[0];
        for (int w = 1; w < SM_WARPS; ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
        am_v = bv;
        am_i = bi;
        chosen = -1;
    }
    cl_sync();
    bv = -INFINITY;
    bi = 0x7fffffff;
    for (unsigned r = 0; r < C; ++r) {
        const float ov = cl_load(&am_v, r);
        const int oi = cl_load(&am_i, r);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }

    int pick = bi;
    bool writer = rank == 0;                               // the CTA that gives the result out
    if (temperature > 0.f) {
        const unsigned long long st = splitmix64((unsigned long long)seeds[row] +
                                                 (unsigned long long)(n_before + 1) * 0x9E3779B97F4A7C15ull);
        const float u = float(st >> 40) * (1.0f / 16777216.0f);
        const float zmax = bv / temperature;
        const bool use_k = top_k > 0 && top_k < V, use_p = top_p < 1.0f;
        // every warp's contiguous piece of the part (a multiple of 32 long), read 32 elements at a time
        const int seg = ((n + SM_WARPS - 1) / SM_WARPS + 31) / 32 * 32;
        const int seg0 = min(n, warp * seg), seg1 = min(n, seg0 + seg);
        const unsigned below = (1u << lane) - 1u;

        if (use_k && top_k <= SM_LIST) {
            // 3. the k-th largest key, eight bits a pass: among the elements whose higher bits equal the prefix
            // found so far, count by the next eight bits and take the bin in which the count from above reaches
            // what is still needed.
            unsigned prefix = 0;
            int need = top_k;
            // Nothing lies above the bin of the largest value: where that bin alone holds top_k elements (the usual
            // case) the first pass is a count of it, without a histogram.
            int first_pass = 0;
            {
                const unsigned top_bin = ordered_key(zmax) >> 24;
                int c = 0;
                for_each_logit(z, n, [&](int, float v) { c += (ordered_key(v) >> 24) == top_bin; });
                c = block_sum<int>(c, is);
                if (tid == 0) cnt_s = c;
                cl_sync();
                int all = 0;
                for (unsigned r = 0; r < C; ++r) all += cl_load(&cnt_s, r);
                if (all >= top_k) {
                    prefix = top_bin << 24;
                    first_pass = 1;
                }
            }
            for (int pass = first_pass; pass < 4; ++pass) {
                const int shift = 24 - 8 * pass;
                int* h = hist[pass & 1];                 // two in turn: the others may still read the last one
                if (tid < 256) h[tid] = 0;
                __syncthreads();
                for_each_logit_in_step(z, n, [&](float v, bool valid) {
                    const unsigned key = ordered_key(v);
                    const bool in = valid && (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8)));
                    if (__ballot_sync(0xffffffffu, in) == 0) return;       // after the first pass few elements are left
                    const int bin = in ? int((key >> shift) & 255u) : -1;
                    // the lanes of a warp that hit the same bin add to it once (most logits share their high bits)
                    const unsigned same = __match_any_sync(0xffffffffu, bin);
                    if (in && lane == __ffs(same) - 1) atomicAdd(&h[bin], __popc(same));
                });
                cl_sync();
                if (tid < 256) {
                    int sum = 0;
                    for (unsigned r = 0; r < C; ++r) sum += cl_load(&h[tid], r);
                    hist_all[tid] = sum;
                }
                __syncthreads();
                if (warp == 0) {
                    int above = 0, b;
                    pick_bin<int>(hist_all, need, lane, b, above);
                    if (lane == 0) {
                        sel_prefix = prefix | (unsigned(b) << shift);
                        sel_need = need - above;
                    }
                }
                __syncthreads();
                prefix = sel_prefix;
                need = sel_need;
            }
            const unsigned tk = prefix;
            const int k_eq = need;                       // of the elements equal to tk, the first k_eq (by index) survive
            // 4. the survivors, in index order, into the first CTA's shared memory: per warp (and per CTA) the
            // number above tk and equal to it ...
            {
                int gt = 0, eq = 0;
                for_each_in_piece(z, seg0, seg1, lane, [&](int, float v, bool inside) {
                    const unsigned key = ordered_key(v);
                    gt += (inside && key > tk);
                    eq += (inside && key == tk);
                    return true;
                });
                for (int o = 16; o > 0; o >>= 1) {
                    gt += __shfl_xor_sync(0xffffffffu, gt, o);
                    eq += __shfl_xor_sync(0xffffffffu, eq, o);
                }
                if (lane == 0) { gt_s[warp] = gt; eq_s[warp] = eq; }
            }
            __syncthreads();
            if (tid == 0) {
                int g = 0, e = 0;
                for (int w = 0; w < SM_WARPS; ++w) { g += gt_s[w]; e += eq_s[w]; }
                tot_gt = g;
                tot_eq = e;
            }
            cl_sync();
            int eq_before = 0, write_at = 0;
            for (unsigned r = 0; r < rank; ++r) {
                const int g = cl_load(&tot_gt, r), e = cl_load(&tot_eq, r);
                write_at += g + max(0, min(e, k_eq - eq_before));
                eq_before += e;
            }
            for (int w = 0; w < warp; ++w) {
                write_at += gt_s[w] + max(0, min(eq_s[w], k_eq - eq_before));
                eq_before += eq_s[w];
            }
            // ... then every warp writes its own at its place
            for_each_in_piece(z, seg0, seg1, lane, [&](int i, float v, bool inside) {
                const unsigned key = ordered_key(v);
                const bool is_eq = inside && key == tk;
                const unsigned eq_mask = __ballot_sync(0xffffffffu, is_eq);
                const bool surv = inside && (key > tk || (is_eq && eq_before + __popc(eq_mask & below) < k_eq));
                const unsigned s_mask = __ballot_sync(0xffffffffu, surv);
                if (surv) {
                    const int at = write_at + __popc(s_mask & below);
                    cl_store(&list_idx[at], 0, lo + i);
                    cl_store(&list_z[at], 0, v);
                }
                write_at += __popc(s_mask);
                eq_before += __popc(eq_mask);
                return true;
            });
            cl_sync();
            if (rank == 0) {
                const int m = top_k;                     // exactly top_k survive
                // 5. the list in descending order (equal values: lower index first): every element counts those before it
                if (tid < m) {
                    const float zj = list_z[tid];
                    const unsigned kj = ordered_key(zj);
                    const float e = expf(zj - zmax);
                    list_e[tid] = e;
                    int before = 0;
                    for (int i = 0; i < m; ++i) {
                        const unsigned ki = ordered_key(list_z[i]);
                        before += (ki > kj) || (ki == kj && i < tid);
                    }
                    sorted_e[before] = e;
                    sorted_pos[before] = short(tid);
                }
                __syncthreads();
                // 6. top_p: the shortest prefix in that order whose mass reaches top_p of the whole (src/sampler.rs:59-69)
                if (tid == 0) {
                    int cut = m;
                    if (use_p) {
                        float Z = 0.f;
                        for (int r = 0; r < m; ++r) Z += sorted_e[r];
                        const float goal = top_p * Z;
                        float cum = 0.f;
                        for (int r = 0; r < m; ++r) {
                            cum += sorted_e[r];
                            if (cum >= goal) { cut = r + 1; break; }
                        }
                    }
                    cut_s = cut;
                }
                __syncthreads();
                if (tid < cut_s) list_idx[sorted_pos[tid]] |= 0x40000000;      // marks the kept ones (indices are below 2^30)
                __syncthreads();
                // 7. the walk over the kept ones in index order
                if (tid == 0) {
                    float Z2 = 0.f;
                    for (int j = 0; j < m; ++j)
                        if (list_idx[j] & 0x40000000) Z2 += list_e[j];
                    const float target = u * Z2;
                    float cum = 0.f;
                    int hit = -1, last = -1;
                    for (int j = 0; j < m; ++j) {
                        if (!(list_idx[j] & 0x40000000)) continue;
                        cum += list_e[j];
                        last = j;
                        if (target < cum) { hit = j; break; }
                    }
                    if (hit < 0) hit = last;                    // the last survivor (src/sampler.rs:78)
                    chosen = hit >= 0 ? (list_idx[hit] & 0x3fffffff) : bi;
                }
                __syncthreads();
                pick = chosen;
            }
        } else if (!use_k) {
            // The whole vocabulary is in play.  3. top_p: the lowest key still inside the nucleus, eight bits a
            // pass as above, but the histogram holds masses; they are summed as 64-bit fixed point (2^-40 of the
            // largest weight), so that a sum does not depend on the order of its terms.
            unsigned tp = 0;
            int p_eq = 0x7fffffff;                       // of the elements equal to tp, the first p_eq (by index) survive
            int eq_before = 0;
            if (use_p) {
                unsigned prefix = 0;
                unsigned long long above = 0, goal = 0;
                for (int pass = 0; pass < 4; ++pass) {
                    const int shift = 24 - 8 * pass;
                    unsigned long long* h = mh[pass & 1];
                    if (tid < 256) h[tid] = 0;
                    __syncthreads();
                    for_each_logit_in_step(z, n, [&](float v, bool valid) {
                        const unsigned key = ordered_key(v);
                        const bool in = valid && (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8)));
                        if (__ballot_sync(0xffffffffu, in) == 0) return;
                        const int bin = in ? int((key >> shift) & 255u) : -1;
                        const unsigned long long m = in ? fixed_mass(v - zmax) : 0ull;
                        // the lanes of a warp that hit the same bin add their masses (41 bits at most, as two halves) once
                        const unsigned same = __match_any_sync(0xffffffffu, bin);
                        const unsigned mlo = __reduce_add_sync(same, unsigned(m & 0xfffffu));
                        const unsigned mhi = __reduce_add_sync(same, unsigned(m >> 20));
                        if (in && lane == __ffs(same) - 1) atomicAdd(&h[bin], ((unsigned long long)mhi << 20) + mlo);
                    });
                    cl_sync();
                    if (tid < 256) {
                        unsigned long long sum = 0;
                        for (unsigned r = 0; r < C; ++r) sum += cl_load(&h[tid], r);
                        mh_all[tid] = sum;
                    }
                    __syncthreads();
                    if (warp == 0) {
                        if (pass == 0) {
                            unsigned long long Z = 0;
                            for (int j = 0; j < 8; ++j) Z += mh_all[8 * lane + j];
                            for (int o = 16; o > 0; o >>= 1) Z += __shfl_xor_sync(0xffffffffu, Z, o);
                            goal = (unsigned long long)(double(top_p) * double(Z));
                            if (goal == 0) goal = 1;
                        }
                        int b;
                        pick_bin<unsigned long long>(mh_all, goal, lane, b, above);
                        if (lane == 0) {
                            sel_goal = goal;
                            sel_prefix = prefix | (unsigned(b) << shift);
                            sel_above = above;
                        }
                    }
                    __syncthreads();
                    prefix = sel_prefix;
                    above = sel_above;
                    goal = sel_goal;
                }
                tp = prefix;
                // every element equal to tp weighs the same: the fewest of them that reach the goal
                const unsigned bits = (tp & 0x80000000u) ? (tp & 0x7fffffffu) : ~tp;
                const unsigned long long e_eq = fixed_mass(__uint_as_float(bits) - zmax);
                if (e_eq > 0 && goal > above) {
                    const unsigned long long c = (goal - above + e_eq - 1) / e_eq;
                    p_eq = c > 0x7ffffffeull ? 0x7fffffff : int(c);
                }
                if (p_eq < 1) p_eq = 1;
                // 4. rank among the elements equal to tp, in index order: how many the pieces (and parts) before hold
                int eq = 0;
                for_each_in_piece(z, seg0, seg1, lane, [&](int, float v, bool inside) {
                    eq += (inside && ordered_key(v) == tp);
                    return true;
                });
                for (int o = 16; o > 0; o >>= 1) eq += __shfl_xor_sync(0xffffffffu, eq, o);
                if (lane == 0) eq_s[warp] = eq;
                __syncthreads();
                if (tid == 0) {
                    int e = 0;
                    for (int w = 0; w < SM_WARPS; ++w) e += eq_s[w];
                    tot_eq = e;
                }
                cl_sync();
                for (unsigned r = 0; r < rank; ++r) eq_before += cl_load(&tot_eq, r);
                for (int w = 0; w < warp; ++w) eq_before += eq_s[w];
            }
            // 5. every warp's mass of survivors, and its last survivor ...
            const bool wide = !use_p;                       // everything survives: no ranks to keep, sums lane by lane
            float cum = 0.f;
            int last = -1, eq_seen = eq_before;
            if (wide) {
                float acc = 0.f;
                for_each_in_piece(z, seg0, seg1, lane, [&](int, float v, bool inside) {
                    acc += inside ? expf(v - zmax) : 0.f;
                    return true;
                });
                cum = __shfl_sync(0xffffffffu, warp_inclusive(acc, lane), 31);
                last = seg1 > seg0 ? lo + seg1 - 1 : -1;
            } else {
                for_each_in_piece(z, seg0, seg1, lane, [&](int i, float v, bool inside) {
                    const unsigned key = ordered_key(v);
                    const unsigned eq_mask = __ballot_sync(0xffffffffu, inside && key == tp);
                    const bool surv = inside && (key > tp || (key == tp && eq_seen + __popc(eq_mask & below) < p_eq));
                    eq_seen += __popc(eq_mask);
                    const float m = surv ? expf(v - zmax) : 0.f;
                    cum += __shfl_sync(0xffffffffu, warp_inclusive(m, lane), 31);
                    const unsigned s_mask = __ballot_sync(0xffffffffu, surv);
                    if (s_mask) last = lo + i - lane + 31 - __clz(s_mask);
                    return true;
                });
            }
            if (lane == 0) { fs[warp] = cum; is[warp] = last; }
            cl_sync();
            // ... 6. the piece in which the target falls, among the pieces of all CTAs ...
            const int pieces = int(C) * SM_WARPS;
            if (tid < pieces) {
                all_m[tid] = cl_load(&fs[tid & 31], unsigned(tid >> 5));
                all_last[tid] = cl_load(&is[tid & 31], unsigned(tid >> 5));
            }
            __syncthreads();
            float Z2 = 0.f;
            int last_all = -1;
            for (int w = 0; w < pieces; ++w) { Z2 += all_m[w]; last_all = max(last_all, all_last[w]); }
            const float target = u * Z2;
            float before = 0.f;
            const int gsel = holder_of(all_m, pieces, target, before);
            writer = gsel < 0 ? rank == 0 : int(rank) == (gsel >> 5);
            if (gsel < 0) {
                pick = last_all >= 0 ? last_all : bi;       // target at or beyond the whole mass (rounding): the last survivor
            } else if (writer) {
                const int wsel = gsel & 31;
                if (wide) {
                    // 7. the piece that holds the target again, every warp with a part of it, and the warp whose
                    // part holds it walks that part, 32 elements at a time in index order
                    const int p0 = min(n, wsel * seg), p1 = min(n, p0 + seg);
                    const int sub = ((p1 - p0 + SM_WARPS - 1) / SM_WARPS + 31) / 32 * 32;
                    const int q0 = min(p1, p0 + warp * sub), q1 = min(p1, q0 + sub);
                    float acc = 0.f;
                    for_each_in_piece(z, q0, q1, lane, [&](int, float v, bool inside) {
                        acc += inside ? expf(v - zmax) : 0.f;
                        return true;
                    });
                    const float tot2 = __shfl_sync(0xffffffffu, warp_inclusive(acc, lane), 31);
                    if (lane == 0) best_v[warp] = tot2;
                    __syncthreads();
                    const int vsel = holder_of(best_v, SM_WARPS, target, before);
                    if (warp == vsel) {
                        float c = before;
                        int hit = -1;
                        for_each_in_piece(z, q0, q1, lane, [&](int i, float v, bool inside) {
                            const float inc = warp_inclusive(inside ? expf(v - zmax) : 0.f, lane);
                            const unsigned mask = __ballot_sync(0xffffffffu, inside && target < c + inc);
                            if (mask) hit = i - lane + __ffs(mask) - 1;
                            c += __shfl_sync(0xffffffffu, inc, 31);
                            return mask == 0;
                        });
                        if (hit < 0) hit = q1 - 1;          // rounding left the target just beyond the part's last element
                        if (lane == 0) chosen = lo + hit;
                    }
                    __syncthreads();
                    pick = chosen >= 0 ? chosen : lo + p1 - 1;
                } else {
                    // 7. the warp whose piece holds the target walks it again
                    if (warp == wsel) {
                        float c = before;
                        int hit = -1;
                        eq_seen = eq_before;
                        for_each_in_piece(z, seg0, seg1, lane, [&](int i, float v, bool inside) {
                            const unsigned key = ordered_key(v);
                            const unsigned eq_mask = __ballot_sync(0xffffffffu, inside && key == tp);
                            const bool surv = inside && (key > tp || (key == tp && eq_seen + __popc(eq_mask & below) < p_eq));
                            eq_seen += __popc(eq_mask);
                            const float inc = warp_inclusive(surv ? expf(v - zmax) : 0.f, lane);
                            const unsigned mask = __ballot_sync(0xffffffffu, surv && target < c + inc);
                            if (mask) hit = lo + i - lane + __ffs(mask) - 1;
                            c += __shfl_sync(0xffffffffu, inc, 31);
                            return mask == 0;
                        });
                        if (hit < 0) hit = last;            // rounding left the target just beyond the piece's last survivor
                        if (lane == 0) chosen = hit;
                    }
                    __syncthreads();
                    pick = chosen >= 0 ? chosen : last_all;
                }
            }
        } else {
            cl_sync();                                      // every part of the row is divided by the temperature
            if (rank == 0) pick = sample_by_bisection(zrow, V, 1.0f, top_k, top_p, zmax, bi, u, fs, is, best_i);
        }
    }
    if (writer && tid == 0) {
        out[row] = pick;
        recent[size_t(slot) * SM_RECENT + (n_before % SM_RECENT)] = pick;
        count[slot] = n_before + 1;
    }
    cl_sync();                                              // nobody leaves while its shared memory may still be read
}

// logits: [n, V] 32-bit, rows ld apart; the penalty is applied to them in place, and with a temperature they
// are left divided by it.
// slots[row] < 0 marks padding.  recent: [slots, 64]; count: [slots].
GB_API int gb_sample(float* logits, long long ld, int n, int V, const int* slots, const long long* seeds,
                     float temperature, int top_k, float top_p, float rep_penalty, int* recent, int* count, int* out,
                     cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && V > 0 && ld >= V, "gb_sample: bad sizes n=%d V=%d ld=%lld", n, V, ld);
    GB_REQUIRE(top_k >= 0 && top_p > 0.f && rep_penalty > 0.f, "gb_sample: bad parameters top_k=%d top_p=%g rep_penalty=%g",
               top_k, top_p, rep_penalty);
    if (n == 0) return 0;
    // CTAs per sequence: as many as leave every CTA 4,096 logits or more and fit the device at once, eight at most
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int cluster = 1;
    while (cluster < SM_MAX_CLUSTER && V / (2 * cluster) >= 4096 && (long long)n * 2 * cluster <= sms) cluster *= 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(n) * cluster);
    cfg.blockDim = dim3(SM_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = unsigned(cluster);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gb_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, sample_kernel, logits, ld, V, slots, seeds, temperature, top_k, top_p, rep_penalty, recent,
                       count, out);
    GB_LAUNCH_OK("gb_sample");
    return 0;
}
