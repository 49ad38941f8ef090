// Embedding gather, residual add + RMS norm, rotation + cache write, gated activation.
// All arithmetic is 32-bit; storage types are chosen by the caller.  Formulas follow the
// reference's CPU forward pass: src/math/ops.rs:1-4 (norm), src/math/rope.rs:6-13
// (rotation), src/model/llama.rs:371-373 (cache write), src/math/ops.rs:11 and
// src/model/llama.rs:401 (gated SiLU).
#include "common.cuh"

// ------------------------------------------------------------------ embedding
__global__ void embed_kernel(const void* __restrict__ table, int table_dtype, const int* __restrict__ tokens,
                             int E, int V, float* __restrict__ out) {
    int t = blockIdx.x;
    int tok = tokens[t];
    float* o = out + size_t(t) * E;
    if (tok < 0 || tok >= V) {
        for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = 0.f;
        return;
    }
    size_t base = size_t(tok) * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = gb_load(table, table_dtype, base + i);
}

// x[t,:] = table[tokens[t],:] as 32-bit floats (the residual stream is kept in 32-bit).
GB_API int gb_embed(const void* table, int table_dtype, const int* tokens, int T, int E, int V, float* out,
                    cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(table_dtype), "gb_embed: bad table dtype %d", table_dtype);
    GB_REQUIRE(T >= 0 && E > 0 && V > 0, "gb_embed: bad sizes T=%d E=%d V=%d", T, E, V);
    if (T == 0) return 0;
    embed_kernel<<<T, 256, 0, stream>>>(table, table_dtype, tokens, E, V, out);
    GB_LAUNCH_OK("gb_embed");
    return 0;
}

// --------------------------------------------------------- add + RMS norm
// For each output row r (source row s = rows ? rows[r] : r):
//   v = x[s,:] + sum_d delta[d][s,:]            (32-bit sum; written back to x when write_x)
//   out[r,:] = v / sqrt(mean(v^2) + eps) * w
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype, int n_delta,
                                   size_t delta_stride, const int* __restrict__ rows, int E,
                                   const void* __restrict__ w, int w_dtype, float eps, void* __restrict__ out,
                                   int out_dtype, int write_x) {
    int r = blockIdx.x;
    int s = rows ? rows[r] : r;
    float* xr = x + size_t(s) * E;
    float ss = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float v = xr[i];
        for (int d = 0; d < n_delta; ++d) v += gb_load(delta, delta_dtype, d * delta_stride + size_t(s) * E + i);
        if (write_x) xr[i] = v;
        ss += v * v;
    }
    __shared__ float red[32];
    __shared__ float total;
    ss = gb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        v = gb_warp_sum(v);
        if (threadIdx.x == 0) total = v;
    }
    __syncthreads();
    float rms = sqrtf(total / float(E) + eps);
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float v = xr[i];
        if (!write_x)
            for (int d = 0; d < n_delta; ++d) v += gb_load(delta, delta_dtype, d * delta_stride + size_t(s) * E + i);
        gb_store(out, out_dtype, size_t(r) * E + i, v / rms * gb_load(w, w_dtype, i));
    }
}

GB_API int gb_add_rmsnorm(float* x, const void* delta, int delta_dtype, int n_delta, long long delta_stride,
                          const int* rows, int n_rows, int E, const void* w, int w_dtype, float eps, void* out,
                          int out_dtype, int write_x, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(w_dtype) && gb_is_dtype(out_dtype), "gb_add_rmsnorm: bad dtype");
    GB_REQUIRE(n_delta == 0 || (delta && gb_is_dtype(delta_dtype)), "gb_add_rmsnorm: bad delta");
    GB_REQUIRE(E > 0 && n_rows >= 0 && eps > 0.f, "gb_add_rmsnorm: bad sizes E=%d rows=%d eps=%g", E, n_rows, eps);
    if (n_rows == 0) return 0;
    int threads = E >= 2048 ? 512 : (E >= 512 ? 256 : 128);
    add_rmsnorm_kernel<<<n_rows, threads, 0, stream>>>(x, delta, delta_dtype, n_delta, size_t(delta_stride), rows, E, w,
                                                       w_dtype, eps, out, out_dtype, write_x);
    GB_LAUNCH_OK("gb_add_rmsnorm");
    return 0;
}

// ------------------------------------------------ rotation + cache write
// One block per token.  q is rotated in place; k is rotated and written to the cache; v
// is copied to the cache.  Angles are position * inv_freq[i] in 32-bit with the
// accurate sincosf.  pairing 0: (i, i + rot/2); pairing 1: (2i, 2i+1).  Dimensions
// beyond rotary_dim pass through.  Tokens of padding (seq_of < 0) are skipped.
constexpr int ROPE_MAX_HALF = 256;

__global__ void rope_kv_write_kernel(void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                                     int dtype, long long ld, int nh, int nkv, int hd, int rotary_dim, int pairing,
                                     const float* __restrict__ inv_freq, const int* __restrict__ seq_of,
                                     const int* __restrict__ pos, const int* __restrict__ table, int table_width,
                                     int ring_pages, void* __restrict__ kcache, void* __restrict__ vcache,
                                     int cache_dtype) {
    int t = blockIdx.x;
    int b = seq_of[t];
    if (b < 0) return;
    int p = pos[t];
    int half = inv_freq ? rotary_dim / 2 : 0;
    __shared__ float sn[ROPE_MAX_HALF], cs[ROPE_MAX_HALF];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float ang = float(p) * inv_freq[i];
        sincosf(ang, &sn[i], &cs[i]);
    }
    __syncthreads();
    size_t row = size_t(t) * size_t(ld);
    if (q) {
        for (int idx = threadIdx.x; idx < nh * half; idx += blockDim.x) {
            int h = idx / half, i = idx - h * half;
            int d0 = pairing ? 2 * i : i, d1 = pairing ? 2 * i + 1 : i + half;
            size_t o = row + size_t(h) * hd;
            float x0 = gb_load(q, dtype, o + d0), x1 = gb_load(q, dtype, o + d1);
            gb_store(q, dtype, o + d0, x0 * cs[i] - x1 * sn[i]);
            gb_store(q, dtype, o + d1, x0 * sn[i] + x1 * cs[i]);
        }
    }
    if (!k) return;
    const int* trow = table + size_t(b) * table_width;
    for (int idx = threadIdx.x; idx < nkv * half; idx += blockDim.x) {
        int g = idx / half, i = idx - g * half;
        int d0 = pairing ? 2 * i : i, d1 = pairing ? 2 * i + 1 : i + half;
        size_t o = row + size_t(g) * hd;
        float x0 = gb_load(k, dtype, o + d0), x1 = gb_load(k, dtype, o + d1);
        size_t c = gb_kv_offset(trow, ring_pages, p, g, nkv, hd);
        gb_store(kcache, cache_dtype, c + d0, x0 * cs[i] - x1 * sn[i]);
        gb_store(kcache, cache_dtype, c + d1, x0 * sn[i] + x1 * cs[i]);
    }
    int rot = 2 * half;
    for (int idx = threadIdx.x; idx < nkv * (hd - rot); idx += blockDim.x) {
        int g = idx / (hd - rot), d = rot + idx - g * (hd - rot);
        size_t c = gb_kv_offset(trow, ring_pages, p, g, nkv, hd);
        gb_store(kcache, cache_dtype, c + d, gb_load(k, dtype, row + size_t(g) * hd + d));
    }
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
        int g = idx / hd, d = idx - g * hd;
        size_t c = gb_kv_offset(trow, ring_pages, p, g, nkv, hd);
        gb_store(vcache, cache_dtype, c + d, gb_load(v, dtype, row + size_t(g) * hd + d));
    }
}

// q, k, v: first elements of the q, k and v parts of token 0's row; rows are `ld` elements
// apart.  k and v may be null (a mixer that reads another run's cache writes none);
// inv_freq may be null (no rotation).
GB_API int gb_rope_kv_write(void* q, const void* k, const void* v, int dtype, long long ld, int T, int nh, int nkv,
                            int hd, int rotary_dim, int pairing, const float* inv_freq, const int* seq_of,
                            const int* pos, const int* table, int table_width, int ring_pages, void* kcache,
                            void* vcache, int cache_dtype, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(cache_dtype), "gb_rope_kv_write: bad dtype");
    GB_REQUIRE(hd > 0 && rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
               "gb_rope_kv_write: rotary_dim %d must be even and at most head_dim %d", rotary_dim, hd);
    GB_REQUIRE(rotary_dim / 2 <= ROPE_MAX_HALF, "gb_rope_kv_write: rotary_dim %d exceeds %d", rotary_dim, 2 * ROPE_MAX_HALF);
    GB_REQUIRE((k == nullptr) == (v == nullptr), "gb_rope_kv_write: k and v must both be given or both be null");
    GB_REQUIRE(!k || (table && kcache && vcache && ring_pages > 0 && table_width >= 1), "gb_rope_kv_write: cache missing");
    if (T == 0) return 0;
    rope_kv_write_kernel<<<T, 128, 0, stream>>>(q, k, v, dtype, ld, nh, nkv, hd, rotary_dim, pairing, inv_freq, seq_of, pos,
                                                table, table_width, ring_pages, kcache, vcache, cache_dtype);
    GB_LAUNCH_OK("gb_rope_kv_write");
    return 0;
}

// ------------------------------------------------------- gated activation
// out[t,i] = silu(gu[t,i]) * gu[t,F+i], silu(z) = z / (1 + exp(-z)).
__global__ void swiglu_kernel(const void* __restrict__ gu, long long ld, void* __restrict__ out, int T, int F, int dtype) {
    size_t n = size_t(T) * F;
    for (size_t idx = blockIdx.x * size_t(blockDim.x) + threadIdx.x; idx < n; idx += size_t(gridDim.x) * blockDim.x) {
        size_t t = idx / F;
        int i = int(idx - t * F);
        float g = gb_load(gu, dtype, t * ld + i), u = gb_load(gu, dtype, t * ld + F + i);
        gb_store(out, dtype, idx, g / (1.f + expf(-g)) * u);
    }
}

GB_API int gb_swiglu(const void* gu, long long ld, void* out, int T, int F, int dtype, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype), "gb_swiglu: bad dtype");
    GB_REQUIRE(F > 0 && T >= 0 && ld >= 2LL * F, "gb_swiglu: bad sizes T=%d F=%d ld=%lld", T, F, ld);
    if (T == 0) return 0;
    size_t n = size_t(T) * F;
    int blocks = int((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    swiglu_kernel<<<blocks, 256, 0, stream>>>(gu, ld, out, T, F, dtype);
    GB_LAUNCH_OK("gb_swiglu");
    return 0;
}
