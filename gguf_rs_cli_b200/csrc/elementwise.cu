// Embedding gather, residual add + RMS norm, rotation + cache write, gated activation.
// All arithmetic is 32-bit; storage types are chosen by the caller.  Formulas follow the
// reference's CPU forward pass: src/math/ops.rs:1-4 (norm), src/math/rope.rs:6-13
// (rotation), src/model/llama.rs:371-373 (cache write), src/math/ops.rs:11 and
// src/model/llama.rs:401 (gated SiLU).
#include "common.cuh"

// ------------------------------------------------------------------ embedding
__global__ void embed_kernel(const void* __restrict__ table, int table_dtype, const int* __restrict__ tokens,
                             int E, int V, float* __restrict__ out) {
    gb_grid_launch_dependents();
    gb_grid_wait();
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
    gb_launch(embed_kernel, dim3(T), dim3(256), 0, stream, table, table_dtype, tokens, E, V, out);
    GB_LAUNCH_OK("gb_embed");
    return 0;
}

// The same, and for the deferred norm of the first layer: xb[t,:] = bf16(x[t,:]) and ssq[t] = sum(x[t,:]^2).
__global__ void embed_shadow_kernel(const void* __restrict__ table, int table_dtype, const int* __restrict__ tokens,
                                    int E, int V, float* __restrict__ out, __nv_bfloat16* __restrict__ xb,
                                    float* __restrict__ ssq) {
    __shared__ float red[32];
    gb_grid_launch_dependents();
    gb_grid_wait();
    int t = blockIdx.x;
    int tok = tokens[t];
    bool ok = tok >= 0 && tok < V;
    size_t base = size_t(ok ? tok : 0) * E;
    float ss = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float v = ok ? gb_load(table, table_dtype, base + i) : 0.f;
        out[size_t(t) * E + i] = v;
        xb[size_t(t) * E + i] = __float2bfloat16_rn(v);
        ss += v * v;
    }
    ss = gb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
        ssq[t] = tot;
    }
}

GB_API int gb_embed_shadow(const void* table, int table_dtype, const int* tokens, int T, int E, int V, float* out,
                           void* xb, float* ssq, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(table_dtype), "gb_embed_shadow: bad table dtype %d", table_dtype);
    GB_REQUIRE(T >= 0 && E > 0 && V > 0 && xb && ssq, "gb_embed_shadow: bad arguments");
    if (T == 0) return 0;
    gb_launch(embed_shadow_kernel, dim3(T), dim3(256), 0, stream, table, table_dtype, tokens, E, V, out, (__nv_bfloat16*)xb, ssq);
    GB_LAUNCH_OK("gb_embed_shadow");
    return 0;
}

// --------------------------------------------------------- add + RMS norm
// For each output row r (source row s = rows ? rows[r] : r):
//   v = x[s,:] + sum_d delta[d][s,:]            (32-bit sum; written back to x when write_x)
//   out[r,:] = v / sqrt(mean(v^2) + eps) * w
// Each thread keeps its share of the row in registers (4 consecutive elements at a time, up
// to NORM_MAX_VEC such groups), so the row is read once; rows too long for that, or not a
// multiple of 4, take the two-pass loop below.
constexpr int NORM_THREADS = 512;
constexpr int NORM_MAX_VEC = 8;          // 512 threads * 8 groups * 4 = rows up to 16384 elements

__device__ __forceinline__ float4 load4(const void* p, int dtype, size_t i) {
    if (dtype == GB_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.x));
    float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(void* p, int dtype, size_t i, float4 v) {
    if (dtype == GB_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v;
    } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned*>(&a);
        raw.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = raw;
    }
}

__device__ __forceinline__ float block_total(float v, float* red) {
    v = gb_warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    return t;
}

template <int NV>
__global__ void __launch_bounds__(NORM_THREADS) add_rmsnorm_vec_kernel(
    float* __restrict__ x, const void* __restrict__ delta, int delta_dtype, int n_delta, size_t delta_stride,
    const int* __restrict__ rows, int E, const void* __restrict__ w, int w_dtype, float eps, void* __restrict__ out,
    int out_dtype, int write_x) {
    __shared__ float red[32];
    gb_grid_launch_dependents();
    gb_grid_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    const size_t base = size_t(s) * E;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int i = (j * NORM_THREADS + threadIdx.x) * 4;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < E) v[j] = *reinterpret_cast<const float4*>(x + base + i);
    }
    for (int d = 0; d < n_delta; ++d) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            int i = (j * NORM_THREADS + threadIdx.x) * 4;
            if (i < E) {
                float4 t = load4(delta, delta_dtype, d * delta_stride + base + i);
                v[j].x += t.x; v[j].y += t.y; v[j].z += t.z; v[j].w += t.w;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    const float rms = sqrtf(block_total(ss, red) / float(E) + eps);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int i = (j * NORM_THREADS + threadIdx.x) * 4;
        if (i < E) {
            if (write_x && n_delta) *reinterpret_cast<float4*>(x + base + i) = v[j];
            float4 wv = load4(w, w_dtype, i);
            store4(out, out_dtype, size_t(r) * E + i,
                   make_float4(v[j].x / rms * wv.x, v[j].y / rms * wv.y, v[j].z / rms * wv.z, v[j].w / rms * wv.w));
        }
    }
}

__global__ void add_rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype, int n_delta,
                                   size_t delta_stride, const int* __restrict__ rows, int E,
                                   const void* __restrict__ w, int w_dtype, float eps, void* __restrict__ out,
                                   int out_dtype, int write_x) {
    __shared__ float red[32];
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
    float rms = sqrtf(block_total(ss, red) / float(E) + eps);
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
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    bool vec = E % 4 == 0 && E <= NORM_THREADS * NORM_MAX_VEC * 4 && aligned(x) && aligned(out) && aligned(w) &&
               (n_delta == 0 || (aligned(delta) && delta_stride % 4 == 0));
#define NORM_LAUNCH(NV)                                                                                              \
    gb_launch(add_rmsnorm_vec_kernel<NV>, dim3(n_rows), dim3(NORM_THREADS), 0, stream, x, delta, delta_dtype, n_delta, \
              size_t(delta_stride), rows, E, w, w_dtype, eps, out, out_dtype, write_x)
    if (vec) {
        int groups = (E / 4 + NORM_THREADS - 1) / NORM_THREADS;
        if (groups <= 1) NORM_LAUNCH(1);
        else if (groups <= 2) NORM_LAUNCH(2);
        else if (groups <= 4) NORM_LAUNCH(4);
        else NORM_LAUNCH(8);
    } else {
        int threads = E >= 2048 ? 512 : (E >= 512 ? 256 : 128);
        add_rmsnorm_kernel<<<n_rows, threads, 0, stream>>>(x, delta, delta_dtype, n_delta, size_t(delta_stride), rows, E, w,
                                                           w_dtype, eps, out, out_dtype, write_x);
    }
#undef NORM_LAUNCH
    GB_LAUNCH_OK("gb_add_rmsnorm");
    return 0;
}

// ------------------------------------------------ rotation + cache write
// One block per (token, group of heads): heads 0..nh-1 of a token are its q heads, rotated in
// place; the next nkv its k heads, rotated into the cache; the last nkv its v heads, copied into
// the cache.  Each thread handles one pair (or two plain elements) of every head of its block;
// few tokens get one head per block (more blocks in flight), many tokens several.  Angles are position * inv_freq[i]
// in 32-bit with the accurate sincosf.  pairing 0: (i, i + rot/2); pairing 1: (2i, 2i+1).
// Dimensions beyond rotary_dim pass through.  Tokens of padding (seq_of < 0) are skipped.
constexpr int ROPE_MAX_HALF = 256;

__global__ void rope_kv_write_kernel(void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                                     int dtype, long long ld, int nh, int nkv, int hd, int rotary_dim, int pairing,
                                     const float* __restrict__ inv_freq, const int* __restrict__ seq_of,
                                     const int* __restrict__ pos, const int* __restrict__ table, int table_width,
                                     int ring_pages, void* __restrict__ kcache, void* __restrict__ vcache,
                                     int cache_dtype, int heads_per_block) {
    gb_grid_launch_dependents();
    gb_grid_wait();
    const int t = blockIdx.x;
    const int b = seq_of[t];
    if (b < 0) return;
    const int p = pos[t];
    const int half = inv_freq ? rotary_dim / 2 : 0;
    const size_t row = size_t(t) * size_t(ld);
    const int i = threadIdx.x;                         // pair index, or element pair index beyond the rotation
    if (i >= hd / 2) return;
    float sn = 0.f, cs = 1.f;
    if (i < half) sincosf(float(p) * inv_freq[i], &sn, &cs);     // one angle serves every head of the block
    const int d0 = i < half ? (pairing ? 2 * i : i) : 2 * i;
    const int d1 = i < half ? (pairing ? 2 * i + 1 : i + half) : 2 * i + 1;
    const int total = k ? nh + 2 * nkv : nh;
    const int head_end = min(total, (blockIdx.y + 1) * heads_per_block);
    const int* trow = k ? table + size_t(b) * table_width : nullptr;
    for (int head = blockIdx.y * heads_per_block; head < head_end; ++head) {
        if (head < nh) {
            if (!q || i >= half) continue;             // q's unrotated dimensions stay as they are
            const size_t o = row + size_t(head) * hd;
            const float x0 = gb_load(q, dtype, o + d0), x1 = gb_load(q, dtype, o + d1);
            float y0, y1;
            gb_rotate(x0, x1, cs, sn, y0, y1);
            gb_store(q, dtype, o + d0, y0);
            gb_store(q, dtype, o + d1, y1);
        } else if (head < nh + nkv) {
            const int g = head - nh;
            const size_t o = row + size_t(g) * hd;
            const size_t c = gb_kv_offset(trow, ring_pages, p, g, nkv, hd);
            const float x0 = gb_load(k, dtype, o + d0), x1 = gb_load(k, dtype, o + d1);
            float y0, y1;
            gb_rotate(x0, x1, cs, sn, y0, y1);                            // beyond the rotation: cs = 1, sn = 0
            gb_store(kcache, cache_dtype, c + d0, y0);
            gb_store(kcache, cache_dtype, c + d1, y1);
        } else {
            const int g = head - nh - nkv;
            const size_t o = row + size_t(g) * hd;
            const size_t c = gb_kv_offset(trow, ring_pages, p, g, nkv, hd);
            gb_store(vcache, cache_dtype, c + 2 * i, gb_load(v, dtype, o + 2 * i));
            gb_store(vcache, cache_dtype, c + 2 * i + 1, gb_load(v, dtype, o + 2 * i + 1));
        }
    }
}

// The same for the common case (bf16 rows and cache, the whole head rotated, pairs (i, i + hd/2), 16-byte
// aligned rows): 16 bytes per load and store.  A thread owns 8 consecutive pair indices (its 8 angles are
// computed once) and walks the q and k heads; then the threads copy v.
constexpr int ROPE_VEC_THREADS = 128;

__global__ void __launch_bounds__(ROPE_VEC_THREADS) rope_kv_write_vec_kernel(
        __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, long long ld,
        int nh, int nkv, int hd, const float* __restrict__ inv_freq, const int* __restrict__ seq_of,
        const int* __restrict__ pos, const int* __restrict__ table, int table_width, int ring_pages,
        __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache) {
    gb_grid_launch_dependents();
    gb_grid_wait();
    const int t = blockIdx.x;
    const int b = seq_of[t];
    if (b < 0) return;
    const int p = pos[t];
    const int half = hd / 2, chunks = hd / 16;             // chunks of 8 pairs per head
    const size_t row = size_t(t) * size_t(ld);
    const int pc = threadIdx.x % chunks, lanes = ROPE_VEC_THREADS / chunks;
    const int* trow = k ? table + size_t(b) * table_width : nullptr;
    if (threadIdx.x < lanes * chunks) {
        float cs[8], sn[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) sincosf(float(p) * inv_freq[8 * pc + i], &sn[i], &cs[i]);
        const int total = k ? nh + nkv : nh;
        for (int head = threadIdx.x / chunks; head < total; head += lanes) {
            const bool is_q = head < nh;
            const __nv_bfloat16* src = is_q ? q + row + size_t(head) * hd : k + row + size_t(head - nh) * hd;
            __nv_bfloat16* dst = is_q ? q + row + size_t(head) * hd
                                      : kcache + gb_kv_offset(trow, ring_pages, p, head - nh, nkv, hd);
            const uint4 lo4 = *reinterpret_cast<const uint4*>(src + 8 * pc);
            const uint4 hi4 = *reinterpret_cast<const uint4*>(src + half + 8 * pc);
            const __nv_bfloat16* lo = reinterpret_cast<const __nv_bfloat16*>(&lo4);
            const __nv_bfloat16* hi = reinterpret_cast<const __nv_bfloat16*>(&hi4);
            uint4 olo4, ohi4;
            __nv_bfloat16* olo = reinterpret_cast<__nv_bfloat16*>(&olo4);
            __nv_bfloat16* ohi = reinterpret_cast<__nv_bfloat16*>(&ohi4);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float y0, y1;
                gb_rotate(__bfloat162float(lo[i]), __bfloat162float(hi[i]), cs[i], sn[i], y0, y1);
                olo[i] = __float2bfloat16_rn(y0);
                ohi[i] = __float2bfloat16_rn(y1);
            }
            *reinterpret_cast<uint4*>(dst + 8 * pc) = olo4;
            *reinterpret_cast<uint4*>(dst + half + 8 * pc) = ohi4;
        }
    }
    if (k) {
        const int per_head = hd / 8;
        for (int idx = threadIdx.x; idx < nkv * per_head; idx += ROPE_VEC_THREADS) {
            const int g = idx / per_head, c = idx - g * per_head;
            *reinterpret_cast<uint4*>(vcache + gb_kv_offset(trow, ring_pages, p, g, nkv, hd) + 8 * c) =
                *reinterpret_cast<const uint4*>(v + row + size_t(g) * hd + 8 * c);
        }
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
    GB_REQUIRE(hd > 0 && hd % 2 == 0 && rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
               "gb_rope_kv_write: head_dim %d and rotary_dim %d must be even, rotary_dim at most head_dim", hd, rotary_dim);
    GB_REQUIRE(hd / 2 <= 1024, "gb_rope_kv_write: head_dim %d exceeds 2048", hd);
    GB_REQUIRE((k == nullptr) == (v == nullptr), "gb_rope_kv_write: k and v must both be given or both be null");
    GB_REQUIRE(!k || (table && kcache && vcache && ring_pages > 0 && table_width >= 1), "gb_rope_kv_write: cache missing");
    GB_REQUIRE(nh + 2 * nkv <= 65535, "gb_rope_kv_write: too many heads");
    if (T == 0) return 0;
    auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    if (dtype == GB_BF16 && (!k || cache_dtype == GB_BF16) && inv_freq && rotary_dim == hd && pairing == 0 && hd % 16 == 0 &&
        hd / 16 <= ROPE_VEC_THREADS && ld % 8 == 0 && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(kcache) &&
        aligned16(vcache) && T >= 64) {
        gb_launch(rope_kv_write_vec_kernel, dim3(T), dim3(ROPE_VEC_THREADS), 0, stream, (__nv_bfloat16*)q,
                  (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, ld, nh, nkv, hd, inv_freq, seq_of, pos, table, table_width,
                  ring_pages, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache);
        GB_LAUNCH_OK("gb_rope_kv_write");
        return 0;
    }
    int threads = ((hd / 2 + 31) / 32) * 32;
    int total = k ? nh + 2 * nkv : nh;
    int heads_per_block = T >= 512 ? 8 : 1;
    dim3 grid(T, (total + heads_per_block - 1) / heads_per_block);
    gb_launch(rope_kv_write_kernel, grid, dim3(threads), 0, stream, q, k, v, dtype, ld, nh, nkv, hd, rotary_dim, pairing, inv_freq,
              seq_of, pos, table, table_width, ring_pages, kcache, vcache, cache_dtype, heads_per_block);
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

// ------------------------------------------------------------- per-slot state
// Zeroes one slot's row in every region of a byte arena: region r starts at table[2r] and holds rows of
// table[2r+1] bytes (a multiple of 4), one per slot.  One block per region.
__global__ void zero_rows_kernel(uint8_t* __restrict__ arena, const long long* __restrict__ table, int slot) {
    const long long off = table[2 * blockIdx.x], row = table[2 * blockIdx.x + 1];
    uint32_t* p = reinterpret_cast<uint32_t*>(arena + off + row * slot);
    for (long long i = threadIdx.x; i < row / 4; i += blockDim.x) p[i] = 0u;
}

// The fixed-size state of a sequence that opens: every state tensor's row `slot` becomes zero in one launch.
GB_API int gb_zero_rows(void* arena, const long long* table, int n_regions, int slot, cudaStream_t stream) {
    GB_REQUIRE(n_regions >= 0 && slot >= 0, "gb_zero_rows: bad sizes regions=%d slot=%d", n_regions, slot);
    if (n_regions == 0) return 0;
    zero_rows_kernel<<<n_regions, 128, 0, stream>>>(reinterpret_cast<uint8_t*>(arena), table, slot);
    GB_LAUNCH_OK("gb_zero_rows");
    return 0;
}
