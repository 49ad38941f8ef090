// Attention for steps in which every sequence brings one token (decode), over the paged
// bf16 cache.  Same arithmetic as the generic kernel (src/model/llama.rs:374-394:
// grouped heads, q.k * scale, softmax with the maximum subtracted, weighted sum of
// values, all in 32-bit) but organised for bandwidth: one CTA per (token, KV head,
// split of the token's pages) serves all query heads of the group from one pass over
// the keys and values, 16-byte loads, four warps on the four quarters of each 64-key
// page.  The splits' partial results (maximum, sum, unnormalised output) go to scratch
// memory; the CTA that arrives last for a (token, KV head) merges them in split order
// and writes the output, so nobody waits and the result does not depend on timing.
//
// Sizes: head_dim a multiple of 16 up to 256, any group size (tiles of up to 8 heads),
// any window.  The grid does not depend on the sequences' lengths (it can be captured
// in a graph): each CTA works out its share of pages from the token's position.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int AD_THREADS = 128;
constexpr int AD_WARPS = 4;
constexpr int AD_KEYS_PER_WARP = GB_PAGE / AD_WARPS;      // 16

struct AdParams {
    const __nv_bfloat16* q;      // [T, nh*hd] rows ldq apart
    __nv_bfloat16* out;          // [T, nh*hd] rows ldo apart
    const __nv_bfloat16* kc;     // [pages, nkv, 64, hd]
    const __nv_bfloat16* vc;
    const int* seq_of;
    const int* pos;
    const int* table;
    float* scratch;              // [T, nh, splits, hd + 2]
    int* counters;               // [T * gridDim.y], zero between launches
    long long ldq, ldo;
    int nh, nkv, hd, table_width, ring_pages, window, splits;
    float scale_log2;            // scale * log2(e)
};

__device__ __forceinline__ void unpack8(uint4 v, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

template <int GT, int HC>
__global__ void __launch_bounds__(AD_THREADS) attention_decode_kernel(AdParams p) {
    gb_grid_launch_dependents();
    gb_grid_wait();
    const int t = blockIdx.x;
    const int G = p.nh / p.nkv;
    const int gtiles = (G + GT - 1) / GT;
    const int g = blockIdx.y / gtiles;                 // KV head
    const int h0 = g * G + (blockIdx.y % gtiles) * GT;  // first query head of this CTA
    const int heads = min(GT, g * G + G - h0);
    const int split = blockIdx.z;
    const int hd = p.hd;
    const int b = p.seq_of[t];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (b < 0) {                                       // padding: zeros, by split 0 only
        if (split == 0)
            for (int i = threadIdx.x; i < heads * hd; i += AD_THREADS)
                p.out[size_t(t) * p.ldo + size_t(h0) * hd + i] = __float2bfloat16_rn(0.f);
        return;
    }

    __shared__ float qs[GT][HC * 64];
    __shared__ float ps[AD_WARPS][GT][AD_KEYS_PER_WARP];
    __shared__ float acc_s[AD_WARPS][GT][HC * 64];
    __shared__ float m_s[AD_WARPS][GT], l_s[AD_WARPS][GT];
    __shared__ int last_flag;

    for (int i = threadIdx.x; i < GT * HC * 64; i += AD_THREADS) {
        int gi = i / (HC * 64), d = i - gi * (HC * 64);
        float v = 0.f;
        if (gi < heads && d < hd) v = __bfloat162float(p.q[size_t(t) * p.ldq + size_t(h0 + gi) * hd + d]) * p.scale_log2;
        qs[gi][d] = v;
    }
    __syncthreads();

    const int pos = p.pos[t];
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int first_page = lo >> GB_PAGE_SHIFT, n_pages = (pos >> GB_PAGE_SHIFT) - first_page + 1;
    const int pg_begin = first_page + int((long long)split * n_pages / p.splits);
    const int pg_end = first_page + int((long long)(split + 1) * n_pages / p.splits);
    const int* trow = p.table + size_t(b) * p.table_width;

    float m[GT], l[GT], acc[GT][HC][2];
#pragma unroll
    for (int gi = 0; gi < GT; ++gi) {
        m[gi] = -INFINITY;
        l[gi] = 0.f;
#pragma unroll
        for (int c = 0; c < HC; ++c) acc[gi][c][0] = acc[gi][c][1] = 0.f;
    }
    const int key_in_warp = lane >> 1, half = lane & 1;
    const int chunks = hd >> 4;                        // 16-byte chunks per lane: the pair of lanes alternates

    for (int pg = pg_begin; pg < pg_end; ++pg) {
        const int phys = trow[pg % p.ring_pages];
        const size_t page_off = (size_t(phys) * p.nkv + g) * GB_PAGE * size_t(hd);
        const int kk = warp * AD_KEYS_PER_WARP + key_in_warp;
        const int j = pg * GB_PAGE + kk;
        const bool valid = j >= lo && j <= pos;
        // ---- scores of this warp's 16 keys; two lanes share a key and take its 16-byte chunks in turn
        float s[GT];
#pragma unroll
        for (int gi = 0; gi < GT; ++gi) s[gi] = 0.f;
        const uint4* kp = reinterpret_cast<const uint4*>(p.kc + page_off + size_t(kk) * hd) + half;
        const float* qh = &qs[0][half * 8];
#pragma unroll 4
        for (int c = 0; c < chunks; ++c) {
            float kf[8];
            unpack8(__ldg(kp + 2 * c), kf);
#pragma unroll
            for (int gi = 0; gi < GT; ++gi) {
                const float* qv = qh + gi * (HC * 64) + c * 16;
#pragma unroll
                for (int e = 0; e < 8; ++e) s[gi] = fmaf(kf[e], qv[e], s[gi]);
            }
        }
        float alpha[GT];
#pragma unroll
        for (int gi = 0; gi < GT; ++gi) {
            float sc = s[gi] + __shfl_xor_sync(0xffffffffu, s[gi], 1);
            sc = valid ? sc : -INFINITY;
            float mx = sc;
#pragma unroll
            for (int o = 2; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            float m_new = fmaxf(m[gi], mx);
            float pj = 0.f;
            alpha[gi] = 1.f;
            if (m_new != -INFINITY) {                  // else: no valid key seen yet, nothing to scale
                alpha[gi] = exp2f(m[gi] - m_new);
                pj = valid ? exp2f(sc - m_new) : 0.f;
            }
            float sum = half == 0 ? pj : 0.f;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            l[gi] = l[gi] * alpha[gi] + sum;
            m[gi] = m_new;
            if (half == 0) ps[warp][gi][key_in_warp] = pj;
        }
        __syncwarp();
        // ---- weighted values: lane owns dimensions 2*lane + 64*c, +1
        const __nv_bfloat16* vp = p.vc + page_off + size_t(warp * AD_KEYS_PER_WARP) * hd;
#pragma unroll
        for (int gi = 0; gi < GT; ++gi)
#pragma unroll
            for (int c = 0; c < HC; ++c) { acc[gi][c][0] *= alpha[gi]; acc[gi][c][1] *= alpha[gi]; }
        const int first_key = pg * GB_PAGE + warp * AD_KEYS_PER_WARP;
#pragma unroll 4
        for (int k = 0; k < AD_KEYS_PER_WARP; ++k) {
            const int jk = first_key + k;
            if (jk < lo || jk > pos) continue;          // uniform over the warp; unwritten rows are never read
            float2 vf[HC];
#pragma unroll
            for (int c = 0; c < HC; ++c) {
                int d = 2 * lane + 64 * c;
                vf[c] = make_float2(0.f, 0.f);
                if (d < hd) vf[c] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vp + size_t(k) * hd + d));
            }
#pragma unroll
            for (int gi = 0; gi < GT; ++gi) {
                float pv = ps[warp][gi][k];
#pragma unroll
                for (int c = 0; c < HC; ++c) {
                    acc[gi][c][0] = fmaf(pv, vf[c].x, acc[gi][c][0]);
                    acc[gi][c][1] = fmaf(pv, vf[c].y, acc[gi][c][1]);
                }
            }
        }
        __syncwarp();
    }

    // ---- merge the four warps in warp order
#pragma unroll
    for (int gi = 0; gi < GT; ++gi) {
#pragma unroll
        for (int c = 0; c < HC; ++c) {
            acc_s[warp][gi][2 * lane + 64 * c] = acc[gi][c][0];
            acc_s[warp][gi][2 * lane + 64 * c + 1] = acc[gi][c][1];
        }
        if (lane == 0) { m_s[warp][gi] = m[gi]; l_s[warp][gi] = l[gi]; }
    }
    __syncthreads();
    const int ytile = blockIdx.y;
    for (int i = threadIdx.x; i < heads * hd; i += AD_THREADS) {
        int gi = i / hd, d = i - gi * hd;
        float M = -INFINITY;
        for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, m_s[w][gi]);
        float L = 0.f, o = 0.f;
        for (int w = 0; w < AD_WARPS; ++w) {
            float wgt = m_s[w][gi] == -INFINITY ? 0.f : exp2f(m_s[w][gi] - M);
            L += l_s[w][gi] * wgt;
            o += acc_s[w][gi][d] * wgt;
        }
        if (p.splits == 1) {
            p.out[size_t(t) * p.ldo + size_t(h0 + gi) * hd + d] = __float2bfloat16_rn(o / L);
        } else {
            float* rec = p.scratch + ((size_t(t) * p.nh + h0 + gi) * p.splits + split) * (hd + 2);
            rec[d] = o;
            if (d == 0) { rec[hd] = M; rec[hd + 1] = L; }
        }
    }
    if (p.splits == 1) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int old = atomicAdd(&p.counters[t * gridDim.y + ytile], 1);
        last_flag = (old == p.splits - 1);
    }
    __syncthreads();
    if (!last_flag) return;                               // the others' records are read from L2 (__ldcg): no fence here
    for (int i = threadIdx.x; i < heads * hd; i += AD_THREADS) {
        int gi = i / hd, d = i - gi * hd;
        const float* rec = p.scratch + (size_t(t) * p.nh + h0 + gi) * p.splits * (hd + 2);
        float M = -INFINITY;
        for (int s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(rec + s * (hd + 2) + hd));
        float L = 0.f, o = 0.f;
        for (int s = 0; s < p.splits; ++s) {
            float ms = __ldcg(rec + s * (hd + 2) + hd);
            float wgt = ms == -INFINITY ? 0.f : exp2f(ms - M);
            L += __ldcg(rec + s * (hd + 2) + hd + 1) * wgt;
            o += __ldcg(rec + s * (hd + 2) + d) * wgt;
        }
        p.out[size_t(t) * p.ldo + size_t(h0 + gi) * hd + d] = __float2bfloat16_rn(o / L);
    }
    if (threadIdx.x == 0) p.counters[t * gridDim.y + ytile] = 0;
}

template <int GT, int HC> int launch_ad(const AdParams& p, dim3 grid, cudaStream_t stream) {
    gb_launch(attention_decode_kernel<GT, HC>, grid, dim3(AD_THREADS), 0, stream, p);
    GB_LAUNCH_OK("gb_attention_decode");
    return 0;
}

template <int GT> int launch_ad_hc(const AdParams& p, dim3 grid, int hc, cudaStream_t stream) {
    switch (hc) {
        case 1: return launch_ad<GT, 1>(p, grid, stream);
        case 2: return launch_ad<GT, 2>(p, grid, stream);
        case 3: return launch_ad<GT, 3>(p, grid, stream);
        default: return launch_ad<GT, 4>(p, grid, stream);
    }
}

int group_tile(int G) { return G >= 8 ? 8 : G > 2 ? 4 : G; }

}  // namespace

GB_API long long gb_attention_decode_scratch_floats(int T, int nh, int hd, int splits) {
    return splits <= 1 ? 0 : (long long)T * nh * splits * (hd + 2);
}

GB_API int gb_attention_decode_supported(int hd, int cache_dtype, int q_dtype) {
    return cache_dtype == GB_BF16 && q_dtype == GB_BF16 && hd >= 16 && hd <= 256 && hd % 16 == 0;
}

// One token per sequence: q [T, nh*hd] bf16 (rotated), cache bf16.  splits chosen by the caller; scratch and counters (T * nkv * group tiles ints, zeroed) are
// needed when splits > 1.
GB_API int gb_attention_decode(const void* q, long long ldq, void* out, long long ldo, int T, int nh, int nkv, int hd,
                               const int* seq_of, const int* pos, const int* table, int table_width, int ring_pages,
                               const void* kcache, const void* vcache, int window, float scale, int splits,
                               float* scratch, int* counters, int n_counters, cudaStream_t stream) {
    GB_REQUIRE(gb_attention_decode_supported(hd, GB_BF16, GB_BF16), "gb_attention_decode: head_dim %d must be a multiple of 16 up to 256", hd);
    GB_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "gb_attention_decode: %d heads are not a multiple of %d KV heads", nh, nkv);
    GB_REQUIRE(window >= 0 && ring_pages > 0 && table_width > 0 && splits >= 1, "gb_attention_decode: bad cache geometry");
    GB_REQUIRE((ldq % 2) == 0 && (ldo % 2) == 0 && (reinterpret_cast<uintptr_t>(kcache) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(vcache) & 15) == 0, "gb_attention_decode: misaligned operands");
    if (T == 0) return 0;
    int G = nh / nkv, gt = group_tile(G), gtiles = (G + gt - 1) / gt;
    GB_REQUIRE(nkv * gtiles <= 65535 && splits <= 65535, "gb_attention_decode: grid too large");
    GB_REQUIRE(splits == 1 || (scratch && counters && (long long)T * nkv * gtiles <= n_counters),
               "gb_attention_decode: splits need scratch and %lld counters", (long long)T * nkv * gtiles);
    AdParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.kc = (const __nv_bfloat16*)kcache;
    p.vc = (const __nv_bfloat16*)vcache; p.seq_of = seq_of; p.pos = pos; p.table = table; p.scratch = scratch;
    p.counters = counters; p.ldq = ldq; p.ldo = ldo; p.nh = nh; p.nkv = nkv; p.hd = hd; p.table_width = table_width;
    p.ring_pages = ring_pages; p.window = window; p.splits = splits; p.scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(T, nkv * gtiles, splits);
    int hc = (hd + 63) / 64;
    switch (gt) {
        case 1: return launch_ad_hc<1>(p, grid, hc, stream);
        case 2: return launch_ad_hc<2>(p, grid, hc, stream);
        case 4: return launch_ad_hc<4>(p, grid, hc, stream);
        default: return launch_ad_hc<8>(p, grid, hc, stream);
    }
}
