// Decode attention (one token per sequence) on the tensor cores, for head sizes 64 and
// 128 over the paged bf16 cache.  The query heads that share a KV head are the rows of
// one 16-row MMA tile (groups larger than 16 take several tiles), so one pass over the
// keys and values serves the whole group with a handful of instructions per page:
// S = Q K^T and O += P V through mma.sync m16n8k16 (bf16 in, f32 accumulate), softmax
// in 32-bit registers.  A CTA is (token, KV head tile, split of the token's pages); its
// 4 warps each take 16 of a page's 64 keys (or its 2 warps 16 of half a page's 32, four
// such CTAs on an SM); pages stream through a 3-stage cp.async ring.  The warps' results
// are merged in warp order, the splits' results by the CTA that arrives last, in split
// order (scratch memory + a counter; nobody waits).
// Same arithmetic as src/model/llama.rs:374-394.  Other head sizes take the CUDA-core
// decode kernel.
#include <math.h>

#include "common.cuh"
#include "stamps.cuh"

namespace {

// Time stamps (builds with -DGB_STAMPS), 16 slots a CTA: 0 entry, 1 the first pages are asked for, 2 the wait for the
// kernel in front is over, 3 the queries are in shared memory, 4 this CTA's first warp has done its pages, 5 all
// warps have, 6 the output (or the split's record) is written.
#ifdef GB_STAMPS
__device__ long long* g_stamps = nullptr;
#define STAMP_IF(cond, k) if (cond) GB_STAMP_WRITE(g_stamps, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, k)
#define STAMP_AFTER_IF(cond, k, val) if (cond) GB_STAMP_WRITE_AFTER(g_stamps, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, k, val)
#else
#define STAMP_IF(cond, k)
#define STAMP_AFTER_IF(cond, k, val)
#endif

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
    // rotation and cache write in the same kernel (rotate != 0): q, k_new and v_new are the products as they
    // come from the projection; the kernel rotates q on its way into shared memory, and the CTA that reads a
    // token's last page puts the token's own rotated key and its value into that page (in shared memory, and
    // one CTA per KV head in the cache too).  k_new null: the cache belongs to another run, only q is rotated.
    int rotate;
    const __nv_bfloat16* k_new;
    const __nv_bfloat16* v_new;
    __nv_bfloat16* kc_w;
    __nv_bfloat16* vc_w;
    const float* inv_freq;
    int rotary_dim, pairing;
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

// The partial results of a (token, head tile)'s splits, merged in split order into the output: every split
// left, per head, its unnormalised sum of values, its maximum (in units of log2) and its sum of weights.
template <int HD>
__device__ __forceinline__ void dm_merge_splits(const DmParams& p, int t, int h0, int heads, int tid, int threads) {
    for (int i = tid; i < heads * HD; i += threads) {
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
}

// WARPS warps take 16 keys each of a unit of WARPS * 16 keys: a whole page with four warps, half a page with two.
// The CTA of two warps needs half the shared memory, so four of them fit an SM where two of the other do: steps
// with more CTAs than fit the device at once in the one shape and no more than fit in the other run in one round.
template <int HD, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) attention_decode_mma_kernel(DmParams p) {
    constexpr int CH = HD / 8, KS = HD / 16, OT = HD / 8, HALF = HD / 2;
    constexpr int THREADS = WARPS * 32, UK = WARPS * 16, UPP = GB_PAGE / UK;      // keys per unit, units per page
    constexpr int PAGE_ELEMS = GB_PAGE * HD, UNIT_ELEMS = UK * HD;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                  // [16][HD]
    __nv_bfloat16* ks = qs + DM_ROWS * HD;                                            // [stages][UK][HD]
    __nv_bfloat16* vs = ks + DM_STAGES * UNIT_ELEMS;                                  // [stages][UK][HD]
    float* merge_o = reinterpret_cast<float*>(ks);                                    // reused after the loop: [WARPS][16][MS]
    constexpr int MS = HD + 8;        // its rows lie 8 banks apart: a warp's 8-byte stores of 8 rows x 4 columns take two passes, not eight
    __shared__ float m_s[WARPS][DM_ROWS], l_s[WARPS][DM_ROWS];
    __shared__ int last_flag;

    // What the kernel in front writes is q (and k_new, v_new).  The index arrays were in place before the step
    // began, and when this kernel writes the token's own key and value itself (rotate with k_new) every row of
    // the cache it reads was written in an earlier step: then the first pages are asked for before waiting for
    // that kernel.  Otherwise the rotation kernel in front wrote the token's row, or (a cache shared with another
    // run) a kernel further back did: wait first.
    STAMP_IF(threadIdx.x == 0, 0);
    gb_grid_launch_dependents();
    const bool early = p.rotate && p.k_new != nullptr;
    if (!early) gb_grid_wait();
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
        if (early) gb_grid_wait();                         // `out` may still be read by a kernel further back
        if (split == 0)
            for (int i = tid; i < heads * HD; i += THREADS)
                p.out[size_t(t) * p.ldo + size_t(h0) * HD + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int pos = p.pos[t];
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int first_page = lo >> GB_PAGE_SHIFT, n_pages = (pos >> GB_PAGE_SHIFT) - first_page + 1;
    const int pg_begin = first_page + int((long long)split * n_pages / p.splits);
    const int pg_end = first_page + int((long long)(split + 1) * n_pages / p.splits);
    // the split's units; those of its pages that lie wholly before the window or behind the token are left out
    const int u_begin = max(pg_begin * UPP, lo / UK), u_end = min(pg_end * UPP, pos / UK + 1);
    const int* trow = p.table + size_t(b) * p.table_width;
    const bool own_kv = p.rotate && p.k_new != nullptr;

    auto load_unit = [&](int u, int stage) {
        const int pg = u / UPP, row0 = (u % UPP) * UK;
        const int phys = trow[pg % p.ring_pages];
        const size_t off = (size_t(phys) * p.nkv + g) * size_t(PAGE_ELEMS) + size_t(row0) * HD;
        __nv_bfloat16* kd = ks + stage * UNIT_ELEMS;
        __nv_bfloat16* vd = vs + stage * UNIT_ELEMS;
        for (int i = tid; i < UK * CH; i += THREADS) {
            int r = i / CH, c = i - r * CH;
            const int key = u * UK + r;                    // rows beyond the sequence are read as zeros, and so
            bool ok = key < pos || (key == pos && !own_kv);   // is the token's own row when this kernel makes it
            dm_cp_async16(kd + dm_swz<HD>(r, c), p.kc + off + size_t(r) * HD + c * 8, ok);
            dm_cp_async16(vd + dm_swz<HD>(r, c), p.vc + off + size_t(r) * HD + c * 8, ok);
        }
    };

    // the group's queries (rows beyond the group are zeros; with the first unit's copies if they need no
    // rotation, else through registers below) and the first units
    if (!p.rotate) {
        for (int i = tid; i < DM_ROWS * CH; i += THREADS) {
            int r = i / CH, c = i - r * CH;
            dm_cp_async16(qs + dm_swz<HD>(r, c), p.q + size_t(t) * p.ldq + size_t(h0 + min(r, heads - 1)) * HD + c * 8, r < heads);
        }
    }
#pragma unroll
    for (int s = 0; s < DM_STAGES - 1; ++s) {
        if (u_begin + s < u_end) load_unit(u_begin + s, s);
        dm_commit();
    }
    // this thread's pairs of every row: pair pi is (pi, pi + half) or (2 pi, 2 pi + 1) inside the rotation,
    // unchanged beyond it; a CTA of fewer threads than pairs gives each thread PPT of them
    constexpr int PPT = HALF > THREADS ? HALF / THREADS : 1;
    constexpr int LANES = HALF / PPT;                      // threads across a row's pairs
    float sn[PPT], cs[PPT];
    int d0[PPT], d1[PPT];
    float own0[PPT], own1[PPT], ownv0[PPT], ownv1[PPT];     // the token's own key and value, this thread's elements
    const bool has_own = own_kv && pg_begin < pg_end && pg_end - 1 == (pos >> GB_PAGE_SHIFT);
#pragma unroll
    for (int e = 0; e < PPT; ++e) { sn[e] = 0.f; cs[e] = 1.f; d0[e] = d1[e] = 0; own0[e] = own1[e] = ownv0[e] = ownv1[e] = 0.f; }
    if (p.rotate) {
        const int half = p.inv_freq ? p.rotary_dim / 2 : 0;
#pragma unroll
        for (int e = 0; e < PPT; ++e) {
            const int pi = tid % LANES + e * LANES;
            const float freq = pi < half ? p.inv_freq[pi] : 0.f;
            d0[e] = pi < half ? (p.pairing ? 2 * pi : pi) : 2 * pi;
            d1[e] = pi < half ? (p.pairing ? 2 * pi + 1 : pi + half) : 2 * pi + 1;
            if (pi < half) sincosf(float(pos) * freq, &sn[e], &cs[e]);
        }
    }
    STAMP_IF(threadIdx.x == 0, 1);
    if (early) gb_grid_wait();                               // the sines and cosines need only the position
    STAMP_IF(threadIdx.x == 0, 2);
    if (p.rotate) {
        constexpr int RSTEP = THREADS / LANES;                   // rows a pass of all threads covers
        constexpr int RPT = DM_ROWS / RSTEP;                     // rows per thread
#pragma unroll
        for (int e = 0; e < PPT; ++e) {
            float x0[RPT], x1[RPT];
#pragma unroll
            for (int j = 0; j < RPT; ++j) {
                const int r = tid / LANES + j * RSTEP;
                x0[j] = x1[j] = 0.f;
                if (r < heads) {
                    const __nv_bfloat16* src = p.q + size_t(t) * p.ldq + size_t(h0 + r) * HD;
                    x0[j] = __bfloat162float(src[d0[e]]);
                    x1[j] = __bfloat162float(src[d1[e]]);
                }
            }
            if (has_own && tid < LANES) {
                const size_t src = size_t(t) * p.ldq + size_t(g) * HD;
                const int pi = tid + e * LANES;
                own0[e] = __bfloat162float(p.k_new[src + d0[e]]);
                own1[e] = __bfloat162float(p.k_new[src + d1[e]]);
                const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(p.v_new + src + 2 * pi);
                ownv0[e] = __low2float(x);
                ownv1[e] = __high2float(x);
            }
#pragma unroll
            for (int j = 0; j < RPT; ++j) {
                const int r = tid / LANES + j * RSTEP;
                float y0, y1;
                gb_rotate(x0[j], x1[j], cs[e], sn[e], y0, y1);
                qs[dm_swz<HD>(r, d0[e] >> 3) + (d0[e] & 7)] = __float2bfloat16_rn(y0);
                qs[dm_swz<HD>(r, d1[e] >> 3) + (d1[e] & 7)] = __float2bfloat16_rn(y1);
            }
        }
    }

    float o[OT][4];
#pragma unroll
    for (int i = 0; i < OT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    unsigned qf[KS][4];
    const int key_base = warp * 16;                          // this warp's 16 keys of every unit

    for (int u = u_begin; u < u_end; ++u) {
        const int it = u - u_begin, stage = it % DM_STAGES;
        if (u + DM_STAGES - 1 < u_end) load_unit(u + DM_STAGES - 1, (it + DM_STAGES - 1) % DM_STAGES);
        dm_commit();
        dm_wait<DM_STAGES - 1>();
        __syncthreads();
        if (has_own && u == pos / UK) {
            // the token's own key (rotated) and value: into the unit in shared memory, and by the first head
            // tile of the KV head into the cache
            const int r = pos & (UK - 1);
            const bool writes = (blockIdx.y % gtiles) == 0;
            const size_t dst = (size_t(trow[(pos >> GB_PAGE_SHIFT) % p.ring_pages]) * p.nkv + g) * size_t(PAGE_ELEMS) +
                               size_t(pos & (GB_PAGE - 1)) * HD;
            if (tid < LANES) {
#pragma unroll
                for (int e = 0; e < PPT; ++e) {
                    float r0, r1;
                    gb_rotate(own0[e], own1[e], cs[e], sn[e], r0, r1);
                    const __nv_bfloat16 y0 = __float2bfloat16_rn(r0), y1 = __float2bfloat16_rn(r1);
                    __nv_bfloat16* kt_w = ks + stage * UNIT_ELEMS;
                    kt_w[dm_swz<HD>(r, d0[e] >> 3) + (d0[e] & 7)] = y0;
                    kt_w[dm_swz<HD>(r, d1[e] >> 3) + (d1[e] & 7)] = y1;
                    const int ev = 2 * (tid + e * LANES);
                    const __nv_bfloat162 x = __floats2bfloat162_rn(ownv0[e], ownv1[e]);
                    __nv_bfloat16* vt_w = vs + stage * UNIT_ELEMS;
                    *reinterpret_cast<__nv_bfloat162*>(vt_w + dm_swz<HD>(r, ev >> 3) + (ev & 7)) = x;
                    if (writes) {
                        p.kc_w[dst + d0[e]] = y0;
                        p.kc_w[dst + d1[e]] = y1;
                        *reinterpret_cast<__nv_bfloat162*>(p.vc_w + dst + ev) = x;
                    }
                }
            }
            __syncthreads();
        }
        STAMP_IF(it == 0 && threadIdx.x == 0, 3);
        if (it == 0) {
#pragma unroll
            for (int k = 0; k < KS; ++k)
                dm_ldmatrix_x4(qf[k][0], qf[k][1], qf[k][2], qf[k][3], qs + dm_swz<HD>(lane & 15, 2 * k + (lane >> 4)));
        }
        const __nv_bfloat16* kt = ks + stage * UNIT_ELEMS;
        const __nv_bfloat16* vt = vs + stage * UNIT_ELEMS;
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
        const int key0 = u * UK + key_base + 2 * (lane & 3);
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
    STAMP_AFTER_IF(threadIdx.x == 0, 4, o[0][0]);
    dm_wait<0>();
    __syncthreads();
    STAMP_IF(threadIdx.x == 0, 5);

    // ---- merge the warps (each saw its share of the keys) in warp order
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    {
        const int ra = lane >> 2, rb = ra + 8, col = 2 * (lane & 3);
        float* mo = merge_o + size_t(warp) * DM_ROWS * MS;
#pragma unroll
        for (int i = 0; i < OT; ++i) {
            if (ra < heads) *reinterpret_cast<float2*>(mo + ra * MS + 8 * i + col) = make_float2(o[i][0], o[i][1]);
            if (rb < heads) *reinterpret_cast<float2*>(mo + rb * MS + 8 * i + col) = make_float2(o[i][2], o[i][3]);
        }
        if ((lane & 3) == 0) {
            m_s[warp][ra] = m0; l_s[warp][ra] = l0;
            m_s[warp][rb] = m1; l_s[warp][rb] = l1;
        }
    }
    __syncthreads();
    for (int i = tid; i < heads * HD; i += THREADS) {
        const int r = i / HD, d = i - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, m_s[w][r]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            float wgt = m_s[w][r] == -INFINITY ? 0.f : exp2f((m_s[w][r] - M) * p.scale_log2);
            L += l_s[w][r] * wgt;
            acc += merge_o[(size_t(w) * DM_ROWS + r) * MS + d] * wgt;
        }
        if (p.splits == 1) {
            p.out[size_t(t) * p.ldo + size_t(h0 + r) * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            float* rec = p.scratch + ((size_t(t) * p.nh + h0 + r) * p.splits + split) * (HD + 2);
            rec[d] = acc;
            if (d == 0) { rec[HD] = M == -INFINITY ? -INFINITY : M * p.scale_log2; rec[HD + 1] = L; }
        }
    }
    STAMP_IF(threadIdx.x == 0, 6);
    if (p.splits == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int old = atomicAdd(&p.counters[t * gridDim.y + blockIdx.y], 1);
        last_flag = (old == p.splits - 1);
    }
    __syncthreads();
    if (!last_flag) return;                               // the others' records are read from L2 (__ldcg): no fence here
    dm_merge_splits<HD>(p, t, h0, heads, tid, THREADS);
    if (tid == 0) p.counters[t * gridDim.y + blockIdx.y] = 0;
}

// The same attention for steps with so few (token, KV head) pairs that the device is mostly idle and a CTA's
// time is the latency of its pages one after the other: twelve warps, each taking quarter pages of 16 keys (warp
// w: quarters w, w + 12, ...) into two slots of shared memory of its own in turn, so that six pages are on their
// way at once, a warp's next quarter arrives while it works on this one, and nobody waits for a block-wide
// barrier per page.  One CTA per SM (24 slots of 16 keys and values); a sequence's pages may be split over
// several CTAs as in the other kernel.
constexpr int PW_WARPS = 12;
constexpr int PW_THREADS = PW_WARPS * 32;
constexpr int PW_KEYS = 16;                 // keys per slot
constexpr int PW_SLOTS = 2;                 // slots per warp
constexpr int PW_UPP = GB_PAGE / PW_KEYS;   // slots' worth of keys per page

template <int HD>
__global__ void __launch_bounds__(PW_THREADS) attention_decode_pages_kernel(DmParams p) {
    constexpr int CH = HD / 8, KS = HD / 16, OT = HD / 8, HALF = HD / 2;
    constexpr int PAGE_ELEMS = GB_PAGE * HD, SLOT_ELEMS = PW_KEYS * HD;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                  // [16][HD]
    __nv_bfloat16* ks = qs + DM_ROWS * HD;                                            // [warps][slots][16][HD]
    __nv_bfloat16* vs = ks + PW_WARPS * PW_SLOTS * SLOT_ELEMS;                        // [warps][slots][16][HD]
    float* merge_o = reinterpret_cast<float*>(ks);                                    // reused after the loop: [warps][16][MS]
    constexpr int MS = HD + 8;        // as in the other kernel
    __shared__ float m_s[PW_WARPS][DM_ROWS], l_s[PW_WARPS][DM_ROWS];
    __shared__ float cs_s[HALF], sn_s[HALF];
    __shared__ int last_flag;

    STAMP_IF(threadIdx.x == 0, 0);
    gb_grid_launch_dependents();
    const bool early = p.rotate && p.k_new != nullptr;       // see the other kernel: pages before the wait
    if (!early) gb_grid_wait();
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
        if (early) gb_grid_wait();
        if (split == 0)
            for (int i = tid; i < heads * HD; i += PW_THREADS)
                p.out[size_t(t) * p.ldo + size_t(h0) * HD + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int pos = p.pos[t];
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int first_page = lo >> GB_PAGE_SHIFT, n_pages = (pos >> GB_PAGE_SHIFT) - first_page + 1;
    const int pg_begin = first_page + int((long long)split * n_pages / p.splits);
    const int pg_end = first_page + int((long long)(split + 1) * n_pages / p.splits);
    const int* trow = p.table + size_t(b) * p.table_width;
    const bool own_kv = p.rotate && p.k_new != nullptr;
    // quarter pages u of the sequence (16 keys each), those of this split's pages that hold a key the token sees
    const int u_first = max(pg_begin * PW_UPP, lo / PW_KEYS), u_end = min(pg_end * PW_UPP, pos / PW_KEYS + 1);

    auto load_quarter = [&](int u, int slot) {
        if (u < u_end) {
            const int pg = u / PW_UPP, row0 = (u % PW_UPP) * PW_KEYS;
            const int phys = trow[pg % p.ring_pages];
            const size_t off = (size_t(phys) * p.nkv + g) * size_t(PAGE_ELEMS) + size_t(row0) * HD;
            __nv_bfloat16* kt = ks + (warp * PW_SLOTS + slot) * SLOT_ELEMS;
            __nv_bfloat16* vt = vs + (warp * PW_SLOTS + slot) * SLOT_ELEMS;
            for (int i = lane; i < PW_KEYS * CH; i += 32) {
                int r = i / CH, c = i - r * CH;
                const int key = u * PW_KEYS + r;               // rows beyond the sequence are read as zeros, and so
                bool ok = key < pos || (key == pos && !own_kv);   // is the token's own row when this kernel makes it
                dm_cp_async16(kt + dm_swz<HD>(r, c), p.kc + off + size_t(r) * HD + c * 8, ok);
                dm_cp_async16(vt + dm_swz<HD>(r, c), p.vc + off + size_t(r) * HD + c * 8, ok);
            }
        }
        dm_commit();                                       // one group per call, also an empty one: the waits count groups
    };
    // every warp's first two quarters are asked for at once
    int u = u_first + warp;
    load_quarter(u, 0);
    load_quarter(u + PW_WARPS, 1);
    // the rotation's cosines and sines, one pair index per thread (the position is known before the kernel in
    // front has finished)
    if (p.rotate && tid < HALF) {
        const int half = p.inv_freq ? p.rotary_dim / 2 : 0;
        float sn = 0.f, cs = 1.f;
        if (tid < half) sincosf(float(pos) * p.inv_freq[tid], &sn, &cs);
        cs_s[tid] = cs;
        sn_s[tid] = sn;
    }
    STAMP_IF(threadIdx.x == 0, 1);
    if (early) gb_grid_wait();
    STAMP_IF(threadIdx.x == 0, 2);

    // the queries
    if (p.rotate) {
        const int half = p.inv_freq ? p.rotary_dim / 2 : 0;
        __syncthreads();
        for (int idx = tid; idx < DM_ROWS * HALF; idx += PW_THREADS) {
            const int r = idx / HALF, pi = idx - r * HALF;
            const int d0 = pi < half ? (p.pairing ? 2 * pi : pi) : 2 * pi;
            const int d1 = pi < half ? (p.pairing ? 2 * pi + 1 : pi + half) : 2 * pi + 1;
            float x0 = 0.f, x1 = 0.f;
            if (r < heads) {
                const __nv_bfloat16* src = p.q + size_t(t) * p.ldq + size_t(h0 + r) * HD;
                x0 = __bfloat162float(src[d0]);
                x1 = __bfloat162float(src[d1]);
            }
            float y0, y1;
            gb_rotate(x0, x1, cs_s[pi], sn_s[pi], y0, y1);
            qs[dm_swz<HD>(r, d0 >> 3) + (d0 & 7)] = __float2bfloat16_rn(y0);
            qs[dm_swz<HD>(r, d1 >> 3) + (d1 & 7)] = __float2bfloat16_rn(y1);
        }
    } else {
        for (int i = tid; i < DM_ROWS * CH; i += PW_THREADS) {
            int r = i / CH, c = i - r * CH;
            dm_cp_async16(qs + dm_swz<HD>(r, c), p.q + size_t(t) * p.ldq + size_t(h0 + min(r, heads - 1)) * HD + c * 8, r < heads);
        }
        dm_commit();
        dm_wait<0>();
    }
    __syncthreads();                                         // the queries are in place
    STAMP_IF(threadIdx.x == 0, 3);

    float o[OT][4];
#pragma unroll
    for (int i = 0; i < OT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    unsigned qf[KS][4];
#pragma unroll
    for (int k = 0; k < KS; ++k)
        dm_ldmatrix_x4(qf[k][0], qf[k][1], qf[k][2], qf[k][3], qs + dm_swz<HD>(lane & 15, 2 * k + (lane >> 4)));

    for (int it = 0; u < u_end; u += PW_WARPS, ++it) {
        const int slot = it & 1;
        __nv_bfloat16* kt = ks + (warp * PW_SLOTS + slot) * SLOT_ELEMS;
        __nv_bfloat16* vt = vs + (warp * PW_SLOTS + slot) * SLOT_ELEMS;
        dm_wait<PW_SLOTS - 1>();                            // all groups but the newest: this quarter is there
        __syncwarp();
        if (own_kv && u == pos / PW_KEYS) {
            // the token's own key (rotated) and value: into the quarter page in shared memory, and by the first
            // head tile of the KV head into the cache
            const int r = pos & (PW_KEYS - 1);
            const int half = p.inv_freq ? p.rotary_dim / 2 : 0;
            const bool writes = (blockIdx.y % gtiles) == 0;
            const size_t src = size_t(t) * p.ldq + size_t(g) * HD;
            const size_t dst = (size_t(trow[(pos >> GB_PAGE_SHIFT) % p.ring_pages]) * p.nkv + g) * size_t(PAGE_ELEMS) +
                               size_t(pos & (GB_PAGE - 1)) * HD;
            for (int pi = lane; pi < HALF; pi += 32) {
                const int d0 = pi < half ? (p.pairing ? 2 * pi : pi) : 2 * pi;
                const int d1 = pi < half ? (p.pairing ? 2 * pi + 1 : pi + half) : 2 * pi + 1;
                float r0, r1;
                gb_rotate(__bfloat162float(p.k_new[src + d0]), __bfloat162float(p.k_new[src + d1]), cs_s[pi], sn_s[pi], r0, r1);
                const __nv_bfloat16 y0 = __float2bfloat16_rn(r0), y1 = __float2bfloat16_rn(r1);
                kt[dm_swz<HD>(r, d0 >> 3) + (d0 & 7)] = y0;
                kt[dm_swz<HD>(r, d1 >> 3) + (d1 & 7)] = y1;
                const int e = 2 * pi;
                const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(p.v_new + src + e);
                *reinterpret_cast<__nv_bfloat162*>(vt + dm_swz<HD>(r, e >> 3) + (e & 7)) = x;
                if (writes) {
                    p.kc_w[dst + d0] = y0;
                    p.kc_w[dst + d1] = y1;
                    *reinterpret_cast<__nv_bfloat162*>(p.vc_w + dst + e) = x;
                }
            }
            __syncwarp();
        }
        // the slot's 16 keys, as the other kernel treats a warp's 16 keys of a page
        {
            constexpr int key_base = 0;
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
            const int key0 = u * PW_KEYS + key_base + 2 * (lane & 3);
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
#pragma unroll
            for (int i2 = 0; i2 < OT / 2; ++i2) {
                unsigned b0, b1, b2, b3;
                dm_ldmatrix_x4_trans(b0, b1, b2, b3, vt + dm_swz<HD>(key_base + (lane & 15), 2 * i2 + (lane >> 4)));
                o[2 * i2][0] *= a0; o[2 * i2][1] *= a0; o[2 * i2][2] *= a1; o[2 * i2][3] *= a1;
                o[2 * i2 + 1][0] *= a0; o[2 * i2 + 1][1] *= a0; o[2 * i2 + 1][2] *= a1; o[2 * i2 + 1][3] *= a1;
                dm_mma(o[2 * i2], pa0, pa1, pa2, pa3, b0, b1);
                dm_mma(o[2 * i2 + 1], pa0, pa1, pa2, pa3, b2, b3);
            }
        }
        __syncwarp();                                        // the slot may be loaded again
        load_quarter(u + PW_SLOTS * PW_WARPS, slot);
    }
    STAMP_AFTER_IF(threadIdx.x == 0, 4, o[0][0]);
    dm_wait<0>();
    __syncthreads();
    STAMP_IF(threadIdx.x == 0, 5);

    // ---- merge the warps (each saw some of the pages) in warp order
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    {
        const int ra = lane >> 2, rb = ra + 8, col = 2 * (lane & 3);
        float* mo = merge_o + size_t(warp) * DM_ROWS * MS;
#pragma unroll
        for (int i = 0; i < OT; ++i) {
            if (ra < heads) *reinterpret_cast<float2*>(mo + ra * MS + 8 * i + col) = make_float2(o[i][0], o[i][1]);
            if (rb < heads) *reinterpret_cast<float2*>(mo + rb * MS + 8 * i + col) = make_float2(o[i][2], o[i][3]);
        }
        if ((lane & 3) == 0) {
            m_s[warp][ra] = m0; l_s[warp][ra] = l0;
            m_s[warp][rb] = m1; l_s[warp][rb] = l1;
        }
    }
    __syncthreads();
    for (int i = tid; i < heads * HD; i += PW_THREADS) {
        const int r = i / HD, d = i - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < PW_WARPS; ++w) M = fmaxf(M, m_s[w][r]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < PW_WARPS; ++w) {
            float wgt = m_s[w][r] == -INFINITY ? 0.f : exp2f((m_s[w][r] - M) * p.scale_log2);
            L += l_s[w][r] * wgt;
            acc += merge_o[(size_t(w) * DM_ROWS + r) * MS + d] * wgt;
        }
        if (p.splits == 1) {
            p.out[size_t(t) * p.ldo + size_t(h0 + r) * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            float* rec = p.scratch + ((size_t(t) * p.nh + h0 + r) * p.splits + split) * (HD + 2);
            rec[d] = acc;
            if (d == 0) { rec[HD] = M == -INFINITY ? -INFINITY : M * p.scale_log2; rec[HD + 1] = L; }
        }
    }
    STAMP_IF(threadIdx.x == 0, 6);
    if (p.splits == 1) return;
    // ---- the splits of a (token, head tile) are merged by the CTA that finishes last, in split order
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int old = atomicAdd(&p.counters[t * gridDim.y + blockIdx.y], 1);
        last_flag = (old == p.splits - 1);
    }
    __syncthreads();
    if (!last_flag) return;                               // the others' records are read from L2 (__ldcg): no fence here
    dm_merge_splits<HD>(p, t, h0, heads, tid, PW_THREADS);
    if (tid == 0) p.counters[t * gridDim.y + blockIdx.y] = 0;
}

template <int HD> int launch_pw(const DmParams& p, dim3 grid, cudaStream_t stream) {
    constexpr int SMEM = (DM_ROWS + 2 * PW_WARPS * PW_SLOTS * PW_KEYS) * HD * 2;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_decode_pages_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return gb_fail("gb_attention_decode_mma: cannot get %d bytes of shared memory", SMEM);
        configured = true;
    }
    gb_launch(attention_decode_pages_kernel<HD>, grid, dim3(PW_THREADS), SMEM, stream, p);
    GB_LAUNCH_OK("gb_attention_decode_mma");
    return 0;
}

template <int HD, int WARPS> int launch_dm(const DmParams& p, dim3 grid, cudaStream_t stream) {
    constexpr int SMEM = (DM_ROWS + 2 * DM_STAGES * WARPS * 16) * HD * 2;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_decode_mma_kernel<HD, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return gb_fail("gb_attention_decode_mma: cannot get %d bytes of shared memory", SMEM);
        configured = true;
    }
    gb_launch(attention_decode_mma_kernel<HD, WARPS>, grid, dim3(WARPS * 32), SMEM, stream, p);
    GB_LAUNCH_OK("gb_attention_decode_mma");
    return 0;
}

}  // namespace

// Builds with -DGB_STAMPS: the CTAs of every decode attention kernel write their time stamps to buf (16 64-bit slots
// a CTA, CTAs in the order of the grid; null: none do).
GB_API int gb_attention_decode_set_stamps(long long* buf) {
#ifdef GB_STAMPS
    if (cudaMemcpyToSymbol(g_stamps, &buf, sizeof(buf)) != cudaSuccess) return gb_fail("gb_attention_decode_set_stamps: cannot set the buffer");
    return 0;
#else
    (void)buf;
    return gb_fail("gb_attention_decode_set_stamps: this library was built without -DGB_STAMPS");
#endif
}

static int g_pages_kernel = 1;        // 0: never the kernel whose warps take whole pages (tuning aid)
GB_API int gb_attention_decode_set_pages_kernel(int on) { g_pages_kernel = on; return 0; }
static int g_two_warps = 1;           // CTAs of two warps: 0 never, 1 by the rule, 2 wherever the head size allows (tuning aid)
GB_API int gb_attention_decode_set_two_warps(int mode) { g_two_warps = mode; return 0; }

GB_API int gb_attention_decode_mma_supported(int hd, int cache_dtype, int q_dtype) {
    return cache_dtype == GB_BF16 && q_dtype == GB_BF16 && (hd == 64 || hd == 128);
}

// Same contract as gb_attention_decode; counters: T * nkv * ceil(G/16) zeroed ints when splits > 1;
// scratch: T * nh * splits * (hd + 2) floats.  With rotate != 0 the kernel also does what gb_rope_kv_write does
// for these tokens: q, k_new, v_new (rows ldq apart, as the projection left them; k_new and v_new null for a
// mixer that reads another run's cache) are rotated by pos * inv_freq (inv_freq null: no rotation) and the
// token's key and value are written at its position of the cache.  q itself stays as it was.
static int decode_mma(const void* q, long long ldq, void* out, long long ldo, int T, int nh, int nkv, int hd,
                      const int* seq_of, const int* pos, const int* table, int table_width, int ring_pages,
                      void* kcache, void* vcache, int window, float scale, int splits, float* scratch,
                      int* counters, int n_counters, int rotate, const void* k_new, const void* v_new,
                      const float* inv_freq, int rotary_dim, int pairing, cudaStream_t stream) {
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
    p.rotate = rotate; p.k_new = (const __nv_bfloat16*)k_new; p.v_new = (const __nv_bfloat16*)v_new;
    p.kc_w = (__nv_bfloat16*)kcache; p.vc_w = (__nv_bfloat16*)vcache; p.inv_freq = inv_freq;
    p.rotary_dim = rotary_dim; p.pairing = pairing;
    dim3 grid(T, nkv * gtiles, splits);
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_pages_kernel && (long long)T * nkv * gtiles * splits <= sms)       // few CTAs: a CTA's latency is the step's
        return hd == 64 ? launch_pw<64>(p, grid, stream) : launch_pw<128>(p, grid, stream);
    // Heads of 128: two CTAs of four warps fit an SM, or four CTAs of two warps.  A step with more CTAs than fit
    // in the first shape, and no more than fit in the second, runs in one round with the second.
    const long long ctas = (long long)T * nkv * gtiles * splits;
    if (hd == 128 && g_two_warps && (g_two_warps == 2 || (ctas > 2LL * sms && ctas <= 4LL * sms)))
        return launch_dm<128, 2>(p, grid, stream);
    return hd == 64 ? launch_dm<64, 4>(p, grid, stream) : launch_dm<128, 4>(p, grid, stream);
}

GB_API int gb_attention_decode_mma(const void* q, long long ldq, void* out, long long ldo, int T, int nh, int nkv, int hd,
                                   const int* seq_of, const int* pos, const int* table, int table_width,
                                   int ring_pages, const void* kcache, const void* vcache, int window, float scale,
                                   int splits, float* scratch, int* counters, int n_counters, cudaStream_t stream) {
    return decode_mma(q, ldq, out, ldo, T, nh, nkv, hd, seq_of, pos, table, table_width, ring_pages, (void*)kcache,
                      (void*)vcache, window, scale, splits, scratch, counters, n_counters, 0, nullptr, nullptr, nullptr,
                      0, 0, stream);
}

GB_API int gb_attention_decode_mma_rope(const void* q, const void* k_new, const void* v_new, long long ldq, void* out,
                                        long long ldo, int T, int nh, int nkv, int hd, int rotary_dim, int pairing,
                                        const float* inv_freq, const int* seq_of, const int* pos, const int* table,
                                        int table_width, int ring_pages, void* kcache, void* vcache, int window,
                                        float scale, int splits, float* scratch, int* counters, int n_counters,
                                        cudaStream_t stream) {
    GB_REQUIRE(rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
               "gb_attention_decode_mma_rope: rotary_dim %d must be even and at most head_dim %d", rotary_dim, hd);
    GB_REQUIRE((k_new == nullptr) == (v_new == nullptr), "gb_attention_decode_mma_rope: k and v must both be given or both be null");
    GB_REQUIRE(!v_new || (reinterpret_cast<uintptr_t>(v_new) & 3) == 0, "gb_attention_decode_mma_rope: misaligned v");
    return decode_mma(q, ldq, out, ldo, T, nh, nkv, hd, seq_of, pos, table, table_width, ring_pages, kcache, vcache,
                      window, scale, splits, scratch, counters, n_counters, 1, k_new, v_new, inv_freq, rotary_dim,
                      pairing, stream);
}
