// Sampling on the device, one block per sequence, in the order of the reference's
// sampler (src/sampler.rs:35-79): repetition penalty on recently emitted tokens;
// temperature <= 0 takes the largest logit; else logits / temperature, the top_k
// largest survive, softmax over them, top_p keeps the smallest set of the most
// probable whose mass reaches it, and one uniform picks a survivor.
//
// Differences from the reference, on purpose: nothing is sorted.  The k-th largest
// value and the top_p cut are found as thresholds by bisection over the ordered bit
// patterns of the floats, ties at a threshold go to the lower indices, and the
// cumulative walk runs over the survivors in index order (the same distribution).
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
constexpr int SM_RECENT = 64;

__device__ __forceinline__ unsigned ordered_key(float z) {
    unsigned u = __float_as_uint(z);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename T> struct SumOp { __device__ T operator()(T a, T b) const { return a + b; } };

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
    __shared__ int chosen;
    gb_grid_launch_dependents();
    gb_grid_wait();
    int row = blockIdx.x, tid = threadIdx.x;
    int slot = slots[row];
    if (slot < 0) {
        if (tid == 0) out[row] = 0;
        return;
    }
    float* z = logits + size_t(row) * ld;
    int n_before = count[slot];

    // 1. repetition penalty, once per occurrence in the ring (src/sampler.rs:23-30)
    if (rep_penalty != 1.0f && tid == 0) {
        int n = min(n_before, SM_RECENT);
        for (int i = 0; i < n; ++i) {
            int tok = recent[size_t(slot) * SM_RECENT + i];
            if (tok >= 0 && tok < V) z[tok] = z[tok] > 0.f ? z[tok] / rep_penalty : z[tok] * rep_penalty;
        }
    }
    __syncthreads();

    // 2. the largest logit and its lowest index
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += SM_THREADS) {
        float v = z[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { best_v[tid >> 5] = bv; best_i[tid >> 5] = bi; }
    __syncthreads();
    bv = best_v[0]; bi = best_i[0];
    for (int w = 1; w < SM_THREADS / 32; ++w)
        if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }

    int pick = bi;
    if (temperature > 0.f) {
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
        unsigned long long st = splitmix64((unsigned long long)seeds[row] +
                                           (unsigned long long)(n_before + 1) * 0x9E3779B97F4A7C15ull);
        float u = float(st >> 40) * (1.0f / 16777216.0f);
        float target = u * Z2;
        if (tid == 0) chosen = -1;
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
        pick = h != 0x7fffffff ? h : (ls >= 0 ? ls : bi);
    }
    if (tid == 0) {
        out[row] = pick;
        recent[size_t(slot) * SM_RECENT + (n_before % SM_RECENT)] = pick;
        count[slot] = n_before + 1;
    }
}

// logits: [n, V] 32-bit, rows ld apart; the penalty is applied to them in place.
// slots[row] < 0 marks padding.  recent: [slots, 64]; count: [slots].
GB_API int gb_sample(float* logits, long long ld, int n, int V, const int* slots, const long long* seeds,
                     float temperature, int top_k, float top_p, float rep_penalty, int* recent, int* count, int* out,
                     cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && V > 0 && ld >= V, "gb_sample: bad sizes n=%d V=%d ld=%lld", n, V, ld);
    GB_REQUIRE(top_k >= 0 && top_p > 0.f && rep_penalty > 0.f, "gb_sample: bad parameters top_k=%d top_p=%g rep_penalty=%g",
               top_k, top_p, rep_penalty);
    if (n == 0) return 0;
    gb_launch(sample_kernel, dim3(n), dim3(SM_THREADS), 0, stream, logits, ld, V, slots, seeds, temperature, top_k, top_p,
              rep_penalty, recent, count, out);
    GB_LAUNCH_OK("gb_sample");
    return 0;
}
