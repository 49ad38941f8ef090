// Attention over the paged cache, one block per (token, query head), for every kind of
// step: whole prompts, continuation and single tokens.  It restates the reference's
// per-head loop (src/model/llama.rs:374-394, src/gpu/attention.glsl:14-77): query head
// h reads KV head h / (nh/nkv); scores q.k * scale over the positions the token may
// see (<= its own, and inside the window if there is one); softmax with the maximum
// subtracted; weighted sum of values.  All in 32-bit with expf.  Keys are taken in
// blocks of 32 absolute positions, warp w taking blocks w, w+4, ..., and the four
// partial results are merged in warp order, so a token's result depends on nothing but
// its own query and keys.  It is the attention of the 32-bit mode, the twin of the
// faster kernels in tests, and the path for head sizes those refuse.
#include <math.h>

#include "common.cuh"

constexpr int AG_MAX_HD = 256;
constexpr int AG_WARPS = 4;

template <typename TC>
__global__ void __launch_bounds__(AG_WARPS * 32) attention_generic_kernel(
    const void* __restrict__ q, int q_dtype, long long ldq, void* __restrict__ out, int out_dtype, long long ldo,
    int nh, int nkv, int hd, const int* __restrict__ seq_of, const int* __restrict__ pos,
    const int* __restrict__ table, int table_width, int ring_pages, const TC* __restrict__ kc,
    const TC* __restrict__ vc, int window, float scale) {
    int t = blockIdx.x, h = blockIdx.y;
    int b = seq_of[t];
    size_t orow = size_t(t) * ldo + size_t(h) * hd;
    if (b < 0) {
        for (int d = threadIdx.x; d < hd; d += blockDim.x) gb_store(out, out_dtype, orow + d, 0.f);
        return;
    }
    __shared__ float qs[AG_MAX_HD];
    __shared__ float acc_s[AG_WARPS][AG_MAX_HD];
    __shared__ float m_s[AG_WARPS], l_s[AG_WARPS];
    for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = gb_load(q, q_dtype, size_t(t) * ldq + size_t(h) * hd + d);
    __syncthreads();

    int p = pos[t];
    int lo = window > 0 ? max(0, p - window + 1) : 0;
    int g = h / (nh / nkv);
    const int* trow = table + size_t(b) * table_width;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int C = AG_MAX_HD / 32;
    float acc[C];
#pragma unroll
    for (int c = 0; c < C; ++c) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int kb = (lo >> 5) + warp; kb <= (p >> 5); kb += AG_WARPS) {
        int j = kb * 32 + lane;
        bool valid = j >= lo && j <= p;
        float s = -INFINITY;
        long long off = 0;
        if (valid) {
            off = (long long)gb_kv_offset(trow, ring_pages, j, g, nkv, hd);
            const TC* kr = kc + off;
            float dot = 0.f;
            for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], gb_to_float(kr[d]), dot);
            s = dot * scale;
        }
        float m_new = fmaxf(m, gb_warp_max(s));
        float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        float pj = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + gb_warp_sum(pj);
#pragma unroll
        for (int c = 0; c < C; ++c) acc[c] *= alpha;
        for (int jj = 0; jj < 32; ++jj) {
            float pv = __shfl_sync(0xffffffffu, pj, jj);
            long long o = __shfl_sync(0xffffffffu, off, jj);
            if (pv != 0.f) {
                const TC* vr = vc + o;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    int d = lane + 32 * c;
                    if (d < hd) acc[c] = fmaf(pv, gb_to_float(vr[d]), acc[c]);
                }
            }
        }
        m = m_new;
    }
#pragma unroll
    for (int c = 0; c < C; ++c) {
        int d = lane + 32 * c;
        if (d < hd) acc_s[warp][d] = acc[c];
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < AG_WARPS; ++w) M = fmaxf(M, m_s[w]);
    float L = 0.f, wgt[AG_WARPS];
    for (int w = 0; w < AG_WARPS; ++w) {
        wgt[w] = (m_s[w] == -INFINITY) ? 0.f : expf(m_s[w] - M);
        L += l_s[w] * wgt[w];
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < AG_WARPS; ++w) o += acc_s[w][d] * wgt[w];
        gb_store(out, out_dtype, orow + d, o / L);
    }
}

// q: [T, nh, hd] with rows ldq elements apart (already rotated); out: [T, nh*hd] with rows ldo
// apart.  seq_of[t] is the token's row in the page table (or -1 for padding, which gives
// zeros), pos[t] its position.  window 0 means all earlier keys.
GB_API int gb_attention_generic(const void* q, int q_dtype, long long ldq, void* out, int out_dtype, long long ldo,
                                int T, int nh, int nkv, int hd, const int* seq_of, const int* pos, const int* table,
                                int table_width, int ring_pages, const void* kcache, const void* vcache,
                                int cache_dtype, int window, float scale, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(q_dtype) && gb_is_dtype(out_dtype) && gb_is_dtype(cache_dtype), "gb_attention_generic: bad dtype");
    GB_REQUIRE(hd > 0 && hd <= AG_MAX_HD, "gb_attention_generic: head_dim %d is not in 1..%d", hd, AG_MAX_HD);
    GB_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "gb_attention_generic: %d heads are not a multiple of %d KV heads", nh, nkv);
    GB_REQUIRE(nh <= 65535, "gb_attention_generic: too many heads (%d)", nh);
    GB_REQUIRE(window >= 0 && ring_pages > 0 && table_width > 0, "gb_attention_generic: bad cache geometry");
    if (T == 0) return 0;
    dim3 grid(T, nh);
    if (cache_dtype == GB_F32)
        attention_generic_kernel<float><<<grid, AG_WARPS * 32, 0, stream>>>(
            q, q_dtype, ldq, out, out_dtype, ldo, nh, nkv, hd, seq_of, pos, table, table_width, ring_pages,
            (const float*)kcache, (const float*)vcache, window, scale);
    else
        attention_generic_kernel<__nv_bfloat16><<<grid, AG_WARPS * 32, 0, stream>>>(
            q, q_dtype, ldq, out, out_dtype, ldo, nh, nkv, hd, seq_of, pos, table, table_width, ring_pages,
            (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, window, scale);
    GB_LAUNCH_OK("gb_attention_generic");
    return 0;
}
