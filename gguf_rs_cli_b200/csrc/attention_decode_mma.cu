// Decode attention (one token per sequence) on the tensor cores, for head sizes 64 and
// 128 over the paged bf16 cache.  The query heads that share a KV head are the rows of
// one 16-row MMA tile (groups larger than 16 take several tiles), so one pass over the
// keys and values serves the whole group with a handful of instructions per page:
// S = Q K^T and O += P V through mma.sync m16n8k16 (bf16 in, f32 accumulate), softmax
// in 32-bit registers.  A CTA is (token, KV head tile, split of the token's pages); its
// 4 warps each take 16 of a page's 64 keys; pages stream through a 3-stage cp.async
// ring.  The warps' results are merged in warp order, the splits' results by the CTA
// that arrives last, in split order (scratch memory + a counter; nobody waits).
// Same arithmetic as src/model/llama.rs:374-394.  Other head sizes take the CUDA-core
// decode kernel.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int DM_THREADS = 128;
constexpr int DM_WARPS = 4;
constexpr int DM_ROWS = 16;           // query heads per tile
constexpr int DM_STAGES = 3;

struct DmParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const __nv_bfloat16* kc;
    const __nv_bfloat16* vc;
    const int* seq_of;
    const int* pos;
    const int* table;
    float* scratch;              // [T, nh, splits, hd + 2]
    int* counters;
    long long ldq, ldo;
    int nh, nkv, table_width, ring_pages, window, splits;
    float scale_log2;
};

__device__ __forceinline__ void dm_cp_async16(void* dst, const void* src, bool valid) {
    unsigned d = unsigned(__cvta_generic_to_shared(dst));
    int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void dm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void dm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void dm_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned a = unsigned(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void dm_ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned a = unsigned(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void dm_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned dm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
template <int HD> __device__ __forceinline__ int dm_swz(int row, int chunk) {
    return row * HD + (((chunk & ~7) | ((chunk ^ row) & 7)) << 3);
}

template <int HD>
__global__ void __launch_bounds__(DM_THREADS) attention_decode_mma_kernel(DmParams p) {
    constexpr int CH = HD / 8, KS = HD / 16, OT = HD / 8;
    constexpr int PAGE_ELEMS = GB_PAGE * HD;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                  // [16][HD]
    __nv_bfloat16* ks = qs + DM_ROWS * HD;                                            // [stages][64][HD]
    __nv_bfloat16* vs = ks + DM_STAGES * PAGE_ELEMS;                                  // [stages][64][HD]
    float* merge_o = reinterpret_cast<float*>(ks);                                    // reused after the loop: [4][16][HD]
    __shared__ float m_s[DM_WARPS][DM_ROWS], l_s[DM_WARPS][DM_ROWS];
    __shared__ int last_flag;

    gb_grid_launch_dependents();
    gb_grid_wait();
    const int t = blockIdx.x;
    const int G = p.nh / p.nkv;
    const int gtiles = (G + DM_ROWS - 1) / DM_ROWS;
    const int g = blockIdx.y / gtiles;
    const int h0 = g * G + (blockIdx.y % gtiles) * DM_ROWS;
    const int heads = min(DM_ROWS, g * G + G - h0);
    const int split = blockIdx.z;
    const int b = p.seq_of[t];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (b < 0) {
        if (split == 0)
            for (int i = tid; i < heads * HD; i += DM_THREADS)
                p.out[size_t(t) * p.ldo + size_t(h0) * HD + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int pos = p.pos[t];
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int first_page = lo >> GB_PAGE_SHIFT, n_pages = (pos >> GB_PAGE_SHIFT) - first_page + 1;
    const int pg_begin = first_page + int((long long)split * n_pages / p.splits);
    const int pg_end = first_page + int((long long)(split + 1) * n_pages / p.splits);
    const int* trow = p.table + size_t(b) * p.table_width;

    auto load_page = [&](int pg, int stage) {
        const int phys = trow[pg % p.ring_pages];
        const size_t off = (size_t(phys) * p.nkv + g) * size_t(PAGE_ELEMS);
        __nv_bfloat16* kd = ks + stage * PAGE_ELEMS;
        __nv_bfloat16* vd = vs + stage * PAGE_ELEMS;
        for (int i = tid; i < GB_PAGE * CH; i += DM_THREADS) {
            int r = i / CH, c = i - r * CH;
            bool ok = pg * GB_PAGE + r <= pos;             // rows beyond the sequence are read as zeros
            dm_cp_async16(kd + dm_swz<HD>(r, c), p.kc + off + size_t(r) * HD + c * 8, ok);
            dm_cp_async16(vd + dm_swz<HD>(r, c), p.vc + off + size_t(r) * HD + c * 8, ok);
        }
    };

    // the group's queries (rows beyond the group are zeros) and the first pages
    for (int i = tid; i < DM_ROWS * CH; i += DM_THREADS) {
        int r = i / CH, c = i - r * CH;
        dm_cp_async16(qs + dm_swz<HD>(r, c), p.q + size_t(t) * p.ldq + size_t(h0 + min(r, heads - 1)) * HD + c * 8, r < heads);
    }
#pragma unroll
    for (int s = 0; s < DM_STAGES - 1; ++s) {
        if (pg_begin + s < pg_end) load_page(pg_begin + s, s);
        dm_commit();
    }

    float o[OT][4];
#pragma unroll
    for (int i = 0; i < OT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    unsigned qf[KS][4];
    const int key_base = warp * 16;                          // this warp's 16 keys of every page

    for (int pg = pg_begin; pg < pg_end; ++pg) {
        const int it = pg - pg_begin, stage = it % DM_STAGES;
        if (pg + DM_STAGES - 1 < pg_end) load_page(pg + DM_STAGES - 1, (it + DM_STAGES - 1) % DM_STAGES);
        dm_commit();
        dm_wait<DM_STAGES - 1>();
        __syncthreads();
        if (it == 0) {
#pragma unroll
            for (int k = 0; k < KS; ++k)
                dm_ldmatrix_x4(qf[k][0], qf[k][1], qf[k][2], qf[k][3], qs + dm_swz<HD>(lane & 15, 2 * k + (lane >> 4)));
        }
        const __nv_bfloat16* kt = ks + stage * PAGE_ELEMS;
        const __nv_bfloat16* vt = vs + stage * PAGE_ELEMS;
        // ---- S[16 heads x 16 keys]
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            unsigned b0, b1, b2, b3;
            dm_ldmatrix_x4(b0, b1, b2, b3, kt + dm_swz<HD>(key_base + (lane & 7) + ((lane >> 4) << 3), 2 * k + ((lane >> 3) & 1)));
            dm_mma(s[0], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b0, b1);
            dm_mma(s[1], qf[k][0], qf[k][1], qf[k][2], qf[k][3], b2, b3);
        }
        // ---- mask (every head sees the same keys) and online softmax; rows lane/4 and lane/4 + 8
        const int key0 = pg * GB_PAGE + key_base + 2 * (lane & 3);
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            int ka = key0 + 8 * j, kb = ka + 1;
            if (ka > pos || ka < lo) s[j][0] = s[j][2] = -INFINITY;
            if (kb > pos || kb < lo) s[j][1] = s[j][3] = -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float a0 = mn0 == -INFINITY ? 1.f : exp2f((m0 - mn0) * p.scale_log2);
        const float a1 = mn1 == -INFINITY ? 1.f : exp2f((m1 - mn1) * p.scale_log2);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0 * p.scale_log2, ms1 = mn1 == -INFINITY ? 0.f : mn1 * p.scale_log2;
        float p00 = exp2f(s[0][0] * p.scale_log2 - ms0), p01 = exp2f(s[0][1] * p.scale_log2 - ms0);
        float p02 = exp2f(s[0][2] * p.scale_log2 - ms1), p03 = exp2f(s[0][3] * p.scale_log2 - ms1);
        float p10 = exp2f(s[1][0] * p.scale_log2 - ms0), p11 = exp2f(s[1][1] * p.scale_log2 - ms0);
        float p12 = exp2f(s[1][2] * p.scale_log2 - ms1), p13 = exp2f(s[1][3] * p.scale_log2 - ms1);
        l0 = l0 * a0 + (p00 + p01 + p10 + p11);
        l1 = l1 * a1 + (p02 + p03 + p12 + p13);
        m0 = mn0;
        m1 = mn1;
        const unsigned pa0 = dm_pack(p00, p01), pa1 = dm_pack(p02, p03), pa2 = dm_pack(p10, p11), pa3 = dm_pack(p12, p13);
        // ---- O += P V over this warp's 16 keys
#pragma unroll
        for (int i2 = 0; i2 < OT / 2; ++i2) {
            unsigned b0, b1, b2, b3;
            dm_ldmatrix_x4_trans(b0, b1, b2, b3, vt + dm_swz<HD>(key_base + (lane & 15), 2 * i2 + (lane >> 4)));
            o[2 * i2][0] *= a0; o[2 * i2][1] *= a0; o[2 * i2][2] *= a1; o[2 * i2][3] *= a1;
            o[2 * i2 + 1][0] *= a0; o[2 * i2 + 1][1] *= a0; o[2 * i2 + 1][2] *= a1; o[2 * i2 + 1][3] *= a1;
            dm_mma(o[2 * i2], pa0, pa1, pa2, pa3, b0, b1);
            dm_mma(o[2 * i2 + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
        __syncthreads();                                    // the stage may be loaded again
    }
    dm_wait<0>();
    __syncthreads();

    // ---- merge the four warps (each saw a quarter of the keys) in warp order
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    {
        const int ra = lane >> 2, rb = ra + 8, col = 2 * (lane & 3);
        float* mo = merge_o + size_t(warp) * DM_ROWS * HD;
#pragma unroll
        for (int i = 0; i < OT; ++i) {
            mo[ra * HD + 8 * i + col] = o[i][0];
            mo[ra * HD + 8 * i + col + 1] = o[i][1];
            mo[rb * HD + 8 * i + col] = o[i][2];
            mo[rb * HD + 8 * i + col + 1] = o[i][3];
        }
        if ((lane & 3) == 0) {
            m_s[warp][ra] = m0; l_s[warp][ra] = l0;
            m_s[warp][rb] = m1; l_s[warp][rb] = l1;
        }
    }
    __syncthreads();
    for (int i = tid; i < heads * HD; i += DM_THREADS) {
        const int r = i / HD, d = i - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DM_WARPS; ++w) M = fmaxf(M, m_s[w][r]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < DM_WARPS; ++w) {
            float wgt = m_s[w][r] == -INFINITY ? 0.f : exp2f((m_s[w][r] - M) * p.scale_log2);
            L += l_s[w][r] * wgt;
            acc += merge_o[(size_t(w) * DM_ROWS + r) * HD + d] * wgt;
        }
        if (p.splits == 1) {
            p.out[size_t(t) * p.ldo + size_t(h0 + r) * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            float* rec = p.scratch + ((size_t(t) * p.nh + h0 + r) * p.splits + split) * (HD + 2);
            rec[d] = acc;
            if (d == 0) { rec[HD] = M == -INFINITY ? -INFINITY : M * p.scale_log2; rec[HD + 1] = L; }
        }
    }
    if (p.splits == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int old = atomicAdd(&p.counters[t * gridDim.y + blockIdx.y], 1);
        last_flag = (old == p.splits - 1);
    }
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    for (int i = tid; i < heads * HD; i += DM_THREADS) {
        const int r = i / HD, d = i - r * HD;
        const float* rec = p.scratch + (size_t(t) * p.nh + h0 + r) * p.splits * (HD + 2);
        float M = -INFINITY;
        for (int s0 = 0; s0 < p.splits; s0 += 8) {
            float mv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) mv[j] = s0 + j < p.splits ? __ldcg(rec + (s0 + j) * (HD + 2) + HD) : -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) M = fmaxf(M, mv[j]);
        }
        float L = 0.f, acc = 0.f;
        for (int s0 = 0; s0 < p.splits; s0 += 8) {
            float mv[8], lv[8], ov[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                bool ok = s0 + j < p.splits;
                mv[j] = ok ? __ldcg(rec + (s0 + j) * (HD + 2) + HD) : -INFINITY;
                lv[j] = ok ? __ldcg(rec + (s0 + j) * (HD + 2) + HD + 1) : 0.f;
                ov[j] = ok ? __ldcg(rec + (s0 + j) * (HD + 2) + d) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float wgt = mv[j] == -INFINITY ? 0.f : exp2f(mv[j] - M);
                L += lv[j] * wgt;
                acc += ov[j] * wgt;
            }
        }
        p.out[size_t(t) * p.ldo + size_t(h0 + r) * HD + d] = __float2bfloat16_rn(acc / L);
    }
    if (tid == 0) p.counters[t * gridDim.y + blockIdx.y] = 0;
}

template <int HD> int launch_dm(const DmParams& p, dim3 grid, cudaStream_t stream) {
    constexpr int SMEM = (DM_ROWS + 2 * DM_STAGES * GB_PAGE) * HD * 2;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_decode_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return gb_fail("gb_attention_decode_mma: cannot get %d bytes of shared memory", SMEM);
        configured = true;
    }
    gb_launch(attention_decode_mma_kernel<HD>, grid, dim3(DM_THREADS), SMEM, stream, p);
    GB_LAUNCH_OK("gb_attention_decode_mma");
    return 0;
}

}  // namespace

GB_API int gb_attention_decode_mma_supported(int hd, int cache_dtype, int q_dtype) {
    return cache_dtype == GB_BF16 && q_dtype == GB_BF16 && (hd == 64 || hd == 128);
}

// Splits of each token's pages for a launch of T tokens (fixed per launch, not per sequence).
GB_API int gb_attention_decode_mma_splits(int T, int nh, int nkv, int sms, int max_pages) {
    int G = nh / nkv, gtiles = (G + DM_ROWS - 1) / DM_ROWS;
    long long ctas = (long long)T * nkv * gtiles;
    int s = int((2LL * sms + ctas - 1) / ctas);
    if (s > max_pages) s = max_pages;
    if (s > 32) s = 32;
    return s < 1 ? 1 : s;
}

// Same contract as gb_attention_decode; counters: T * nkv * ceil(G/16) zeroed ints when splits > 1;
// scratch: T * nh * splits * (hd + 2) floats.
GB_API int gb_attention_decode_mma(const void* q, long long ldq, void* out, long long ldo, int T, int nh, int nkv, int hd,
                                   const int* seq_of, const int* pos, const int* table, int table_width,
                                   int ring_pages, const void* kcache, const void* vcache, int window, float scale,
                                   int splits, float* scratch, int* counters, int n_counters, cudaStream_t stream) {
    GB_REQUIRE(gb_attention_decode_mma_supported(hd, GB_BF16, GB_BF16), "gb_attention_decode_mma: head_dim %d is not 64 or 128", hd);
    GB_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "gb_attention_decode_mma: %d heads are not a multiple of %d KV heads", nh, nkv);
    GB_REQUIRE(window >= 0 && ring_pages > 0 && table_width > 0 && splits >= 1, "gb_attention_decode_mma: bad cache geometry");
    GB_REQUIRE((ldq % 8) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(kcache) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(vcache) & 15) == 0, "gb_attention_decode_mma: misaligned operands");
    if (T == 0) return 0;
    int G = nh / nkv, gtiles = (G + DM_ROWS - 1) / DM_ROWS;
    GB_REQUIRE(nkv * gtiles <= 65535 && splits <= 65535, "gb_attention_decode_mma: grid too large");
    GB_REQUIRE(splits == 1 || (scratch && counters && (long long)T * nkv * gtiles <= n_counters),
               "gb_attention_decode_mma: splits need scratch and %lld counters", (long long)T * nkv * gtiles);
    DmParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.kc = (const __nv_bfloat16*)kcache;
    p.vc = (const __nv_bfloat16*)vcache; p.seq_of = seq_of; p.pos = pos; p.table = table; p.scratch = scratch;
    p.counters = counters; p.ldq = ldq; p.ldo = ldo; p.nh = nh; p.nkv = nkv; p.table_width = table_width;
    p.ring_pages = ring_pages; p.window = window; p.splits = splits; p.scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(T, nkv * gtiles, splits);
    return hd == 64 ? launch_dm<64>(p, grid, stream) : launch_dm<128>(p, grid, stream);
}
