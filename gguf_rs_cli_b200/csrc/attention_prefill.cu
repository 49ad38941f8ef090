// Attention for steps that bring many tokens per sequence (prompts and their further
// pieces), over the paged bf16 cache, which already holds this step's keys and values.
// Same arithmetic as the generic kernel (src/model/llama.rs:374-394) in flash form: a
// CTA owns 128 consecutive queries of one sequence and one head, walks the sequence's
// pages (64 keys each) up to the causal limit, keeps running maxima and sums per query
// in 32-bit and never materialises the score matrix.  Products run on the tensor
// cores through mma.sync m16n8k16 (bf16 in, f32 accumulate): 8 warps x 16 queries;
// K and V pages are double-buffered in shared memory with cp.async.
//
// Sizes: head_dim 64 or 128 here (other sizes take the generic kernel), any group
// size, any window, sequences that start anywhere in their cache.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int AP_BM = 128;          // queries per CTA
constexpr int AP_BN = GB_PAGE;      // keys per step = one page
constexpr int AP_WARPS = 8;
constexpr int AP_THREADS = AP_WARPS * 32;

struct ApParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const __nv_bfloat16* kc;
    const __nv_bfloat16* vc;
    const int* tiles;      // [n_tiles][2]: sequence row, first query of the tile within this step's tokens of it
    const int* cu;         // [B+1] first packed token of each sequence
    const int* starts;     // [B] cached length before this step
    const int* qlens;      // [B]
    const int* table;
    long long ldq, ldo;
    int nh, nkv, table_width, ring_pages, window;
    float scale_log2;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    unsigned d = unsigned(__cvta_generic_to_shared(dst));
    int n = valid ? 16 : 0;                       // 0 source bytes: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned a = unsigned(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned a = unsigned(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Element offset of (row, 16-byte chunk) in a tile of HD-wide bf16 rows whose chunks are
// XOR-swizzled within groups of 8 so that ldmatrix rows fall into distinct banks.
template <int HD> __device__ __forceinline__ int swz(int row, int chunk) {
    return row * HD + (((chunk & ~7) | ((chunk ^ row) & 7)) << 3);
}

template <int HD>
__global__ void __launch_bounds__(AP_THREADS, 2) attention_prefill_kernel(ApParams p) {
    constexpr int CH = HD / 8;            // 16-byte chunks per row
    constexpr int KS = HD / 16;           // k-steps of Q.K^T
    constexpr int NT = AP_BN / 8;         // score n-tiles per warp (8 keys each)
    constexpr int OT = HD / 8;            // output n-tiles
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [128][HD]
    __nv_bfloat16* ks = qs + AP_BM * HD;                                       // [2][64][HD]
    __nv_bfloat16* vs = ks + 2 * AP_BN * HD;                                   // [2][64][HD]

    gb_grid_launch_dependents();
    gb_grid_wait();
    // blockIdx.x (which varies fastest in the order CTAs start) is the head, blockIdx.y the tile: all heads of
    // the first tile in the caller's list start before any head of the second
    const int b = p.tiles[2 * blockIdx.y], q0 = p.tiles[2 * blockIdx.y + 1];
    const int h = blockIdx.x, g = h / (p.nh / p.nkv);
    const int start = p.starts[b], qlen = p.qlens[b], tok0 = p.cu[b] + q0;
    const int rows = min(AP_BM, qlen - q0);                   // valid queries of this tile
    const int last_pos = start + qlen - 1;                    // last position the cache holds for this sequence
    const int* trow = p.table + size_t(b) * p.table_width;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // key pages this tile needs
    const int pos_lo = start + q0, pos_hi = start + q0 + rows - 1;
    const int kb_begin = p.window > 0 ? max(0, pos_lo - p.window + 1) >> GB_PAGE_SHIFT : 0;
    const int kb_end = (pos_hi >> GB_PAGE_SHIFT) + 1;

    auto load_kv = [&](int kb, int buf) {
        const int phys = trow[kb % p.ring_pages];
        const size_t off = (size_t(phys) * p.nkv + g) * AP_BN * size_t(HD);
        __nv_bfloat16* kd = ks + buf * AP_BN * HD;
        __nv_bfloat16* vd = vs + buf * AP_BN * HD;
        for (int i = tid; i < AP_BN * CH; i += AP_THREADS) {
            int r = i / CH, c = i - r * CH;
            bool ok = kb * AP_BN + r <= last_pos;              // rows never written are read as zeros
            cp_async16(kd + swz<HD>(r, c), p.kc + off + size_t(r) * HD + c * 8, ok);
            cp_async16(vd + swz<HD>(r, c), p.vc + off + size_t(r) * HD + c * 8, ok);
        }
    };

    // Q tile and the first K/V page
    for (int i = tid; i < AP_BM * CH; i += AP_THREADS) {
        int r = i / CH, c = i - r * CH;
        cp_async16(qs + swz<HD>(r, c), p.q + size_t(tok0 + min(r, rows - 1)) * p.ldq + size_t(h) * HD + c * 8, r < rows);
    }
    load_kv(kb_begin, 0);
    cp_async_commit();

    // this thread's two query rows and their positions (-1: no such query)
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int pq0 = r0 < rows ? start + q0 + r0 : -1, pq1 = r1 < rows ? start + q0 + r1 : -1;
    const int lo0 = p.window > 0 ? pq0 - p.window + 1 : 0, lo1 = p.window > 0 ? pq1 - p.window + 1 : 0;

    float o[OT][4];
#pragma unroll
    for (int i = 0; i < OT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int buf = (kb - kb_begin) & 1;
        if (kb + 1 < kb_end) load_kv(kb + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* kt = ks + buf * AP_BN * HD;
        const __nv_bfloat16* vt = vs + buf * AP_BN * HD;

        // ---- S = Q K^T for 16 queries x 64 keys
        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            // the query fragment is read from shared memory at every step: holding all of Q in registers
            // would leave room for one CTA per SM only
            unsigned qf[4];
            ldmatrix_x4(qf[0], qf[1], qf[2], qf[3], qs + swz<HD>(warp * 16 + (lane & 15), 2 * k + (lane >> 4)));
#pragma unroll
            for (int j2 = 0; j2 < NT / 2; ++j2) {
                unsigned b0, b1, b2, b3;
                // keys 16*j2 .. +15; lanes 0-7 / 8-15 / 16-23 / 24-31 address (keys 0-7, d lo), (keys 0-7, d hi),
                // (keys 8-15, d lo), (keys 8-15, d hi)
                ldmatrix_x4(b0, b1, b2, b3, kt + swz<HD>(j2 * 16 + (lane & 7) + ((lane >> 4) << 3), 2 * k + ((lane >> 3) & 1)));
                mma_bf16(s[2 * j2], qf[0], qf[1], qf[2], qf[3], b0, b1);
                mma_bf16(s[2 * j2 + 1], qf[0], qf[1], qf[2], qf[3], b2, b3);
            }
        }
        // ---- mask and online softmax (two rows per thread: r0 in c0,c1 and r1 in c2,c3)
        const int key0 = kb * AP_BN + 2 * (lane & 3);
        const bool need_mask = (kb * AP_BN + AP_BN - 1 > pos_lo) || (p.window > 0);
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            if (need_mask) {
                int ka = key0 + 8 * j, kb2 = ka + 1;
                if (ka > pq0 || ka < lo0) s[j][0] = -INFINITY;
                if (kb2 > pq0 || kb2 < lo0) s[j][1] = -INFINITY;
                if (ka > pq1 || ka < lo1) s[j][2] = -INFINITY;
                if (kb2 > pq1 || kb2 < lo1) s[j][3] = -INFINITY;
            }
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
        float sum0 = 0.f, sum1 = 0.f;
        unsigned pf[NT][2];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            float p0 = exp2f(s[j][0] * p.scale_log2 - ms0), p1 = exp2f(s[j][1] * p.scale_log2 - ms0);
            float p2 = exp2f(s[j][2] * p.scale_log2 - ms1), p3 = exp2f(s[j][3] * p.scale_log2 - ms1);
            sum0 += p0 + p1;
            sum1 += p2 + p3;
            pf[j][0] = pack_bf16(p0, p1);
            pf[j][1] = pack_bf16(p2, p3);
        }
        l0 = l0 * a0 + sum0;
        l1 = l1 * a1 + sum1;
        m0 = mn0;
        m1 = mn1;
#pragma unroll
        for (int i = 0; i < OT; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < AP_BN / 16; ++kk) {
#pragma unroll
            for (int i2 = 0; i2 < OT / 2; ++i2) {
                unsigned b0, b1, b2, b3;
                // keys 16*kk .. +15, dims 16*i2 .. +15, transposed: lanes 0-7 / 8-15 / 16-23 / 24-31 address
                // (keys 0-7, d lo), (keys 8-15, d lo), (keys 0-7, d hi), (keys 8-15, d hi)
                ldmatrix_x4_trans(b0, b1, b2, b3, vt + swz<HD>(kk * 16 + (lane & 15), 2 * i2 + (lane >> 4)));
                mma_bf16(o[2 * i2], pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1], b0, b1);
                mma_bf16(o[2 * i2 + 1], pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1], b2, b3);
            }
        }
        __syncthreads();            // everyone is done with this buffer before it is loaded again
    }
    cp_async_wait<0>();

    // ---- normalise and store
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    __nv_bfloat16* out0 = p.out + size_t(tok0 + r0) * p.ldo + size_t(h) * HD + 2 * (lane & 3);
    __nv_bfloat16* out1 = p.out + size_t(tok0 + r1) * p.ldo + size_t(h) * HD + 2 * (lane & 3);
#pragma unroll
    for (int i = 0; i < OT; ++i) {
        if (r0 < rows) *reinterpret_cast<__nv_bfloat162*>(out0 + 8 * i) = __floats2bfloat162_rn(o[i][0] * inv0, o[i][1] * inv0);
        if (r1 < rows) *reinterpret_cast<__nv_bfloat162*>(out1 + 8 * i) = __floats2bfloat162_rn(o[i][2] * inv1, o[i][3] * inv1);
    }
}

template <int HD> int launch_ap(const ApParams& p, int n_tiles, cudaStream_t stream) {
    constexpr int SMEM = (AP_BM + 4 * AP_BN) * HD * 2;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return gb_fail("gb_attention_prefill: cannot get %d bytes of shared memory", SMEM);
        configured = true;
    }
    gb_launch(attention_prefill_kernel<HD>, dim3(p.nh, n_tiles), dim3(AP_THREADS), SMEM, stream, p);
    GB_LAUNCH_OK("gb_attention_prefill");
    return 0;
}

}  // namespace

GB_API int gb_attention_prefill_supported(int hd, int cache_dtype, int q_dtype) {
    return cache_dtype == GB_BF16 && q_dtype == GB_BF16 && (hd == 64 || hd == 128);
}

// Queries per tile: the caller lists, for every sequence of the step, tiles (sequence row, first query)
// in steps of this many queries.
GB_API int gb_attention_prefill_tile() { return AP_BM; }

GB_API int gb_attention_prefill(const void* q, long long ldq, void* out, long long ldo, int nh, int nkv, int hd,
                                const int* tiles, int n_tiles, const int* cu, const int* starts, const int* qlens,
                                const int* table, int table_width, int ring_pages, const void* kcache,
                                const void* vcache, int window, float scale, cudaStream_t stream) {
    GB_REQUIRE(gb_attention_prefill_supported(hd, GB_BF16, GB_BF16), "gb_attention_prefill: head_dim %d is not 64 or 128", hd);
    GB_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "gb_attention_prefill: bad head counts %d / %d", nh, nkv);
    GB_REQUIRE(n_tiles <= 65535, "gb_attention_prefill: %d tiles of queries are too many for one launch", n_tiles);
    GB_REQUIRE(window >= 0 && ring_pages > 0 && table_width > 0, "gb_attention_prefill: bad cache geometry");
    GB_REQUIRE((ldq % 8) == 0 && (ldo % 2) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(kcache) & 15) == 0 && (reinterpret_cast<uintptr_t>(vcache) & 15) == 0,
               "gb_attention_prefill: misaligned operands");
    if (n_tiles == 0) return 0;
    ApParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.kc = (const __nv_bfloat16*)kcache;
    p.vc = (const __nv_bfloat16*)vcache; p.tiles = tiles; p.cu = cu; p.starts = starts; p.qlens = qlens; p.table = table;
    p.ldq = ldq; p.ldo = ldo; p.nh = nh; p.nkv = nkv; p.table_width = table_width; p.ring_pages = ring_pages;
    p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
    return hd == 64 ? launch_ap<64>(p, n_tiles, stream) : launch_ap<128>(p, n_tiles, stream);
}
