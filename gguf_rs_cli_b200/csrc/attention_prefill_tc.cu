// Attention for prompts on the 5th-generation tensor cores (head size 128): the same
// arithmetic as attention_prefill.cu and the generic kernel (src/model/llama.rs:374-394),
// with both products of flash attention issued as tcgen05.mma and their results in TMEM.
//
// A CTA owns 128 consecutive queries of one sequence and one head and walks the keys in
// blocks of 128 (two cache pages).  10 warps:
//   warp 0  TMA: Q once, then K and V pages into two-stage rings (128-byte swizzle);
//   warp 1  one thread issues S = Q K^T (M128 N128 K128) into one of two TMEM buffers and,
//           when the probabilities are ready, O += P V (P is read from TMEM, V from shared memory
//           N-contiguous, as the cache stores it) into the output accumulator, which stays in TMEM
//           for the whole tile;
//   warps 2-9  two threads per query row (its TMEM lane), each with 64 of a block's 128 keys: read S,
//           mask, maximum (agreed between the two through shared memory) and sum in 32-bit, write P as
//           bf16 into one of two TMEM buffers (the A operand of the second product).
//           Probabilities are taken relative to a reference maximum that is only raised when
//           the row's maximum has grown by more than 2^8; only then is the row of O in TMEM
//           (and the running sum) rescaled, so most blocks touch O through the MMA alone.
// All hand-overs are mbarriers; every wait is bounded and reports through the status word.
// Rows of a page beyond the sequence's end are zeroed in shared memory before they are
// multiplied (they were never written and may hold anything).
#include <math.h>

#include "common.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int AT_BM = 128, AT_BN = 128, AT_HD = 128;
constexpr int AT_THREADS = 320;          // TMA, MMA and eight softmax warps
constexpr int AT_CHUNK = 128 * 128;            // bytes of a [128 rows x 64 columns] bf16 tile
constexpr int AT_TILE = 2 * AT_CHUNK;          // 32 KB: 128 x 128 bf16
constexpr int AT_PAGE_CHUNK = 64 * 128;        // bytes of a [64 rows x 64 columns] piece of a page
constexpr int AT_SMEM = 5 * AT_TILE + 1024;    // Q, K x2, V x2 (+ alignment slack)
constexpr int AT_TMEM_COLS = 512;              // S x2 (128 each), O (128), P x2 (64 each: 128 bf16 a row)

struct AtParams {
    __nv_bfloat16* out;
    const int* tiles;
    const int* cu;
    const int* starts;
    const int* qlens;
    const int* table;
    int* status;
    long long ldo;
    int nh, nkv, table_width, ring_pages, window;
    float scale_log2;
};

__device__ __forceinline__ uint4 pack8(const float* p) {
    __nv_bfloat162 a = __floats2bfloat162_rn(p[0], p[1]), b = __floats2bfloat162_rn(p[2], p[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(p[4], p[5]), d = __floats2bfloat162_rn(p[6], p[7]);
    uint4 r;
    r.x = *reinterpret_cast<unsigned*>(&a);
    r.y = *reinterpret_cast<unsigned*>(&b);
    r.z = *reinterpret_cast<unsigned*>(&c);
    r.w = *reinterpret_cast<unsigned*>(&d);
    return r;
}

__global__ void __launch_bounds__(AT_THREADS, 1) attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                             const __grid_constant__ CUtensorMap map_k,
                                                                             const __grid_constant__ CUtensorMap map_v,
                                                                             AtParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = base;
    uint8_t* k_s = base + AT_TILE;               // 2 stages
    uint8_t* v_s = base + 3 * AT_TILE;           // 2 stages
    __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full[2], p_empty[2];
    __shared__ uint32_t tmem_base;
    __shared__ volatile int abort_flag;
    __shared__ float mx_s[2][2][AT_BM], l_s[2][AT_BM];      // exchanged between the two threads of a query row

    gb_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = p.tiles[2 * blockIdx.y], q0 = p.tiles[2 * blockIdx.y + 1];
    const int h = blockIdx.x, g = h / (p.nh / p.nkv);
    const int start = p.starts[b], qlen = p.qlens[b], tok0 = p.cu[b] + q0;
    const int rows = min(AT_BM, qlen - q0);
    const int last_pos = start + qlen - 1;
    const int pos_lo = start + q0, pos_hi = pos_lo + rows - 1;
    const int pg_begin = p.window > 0 ? max(0, pos_lo - p.window + 1) >> GB_PAGE_SHIFT : 0;
    const int pg_end = (pos_hi >> GB_PAGE_SHIFT) + 1;
    const int n_blocks = (pg_end - pg_begin + 1) / 2;
    const int valid_end = min(last_pos, pg_end * GB_PAGE - 1);   // last key position that was both written and loaded
    const int* trow = p.table + size_t(b) * p.table_width;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 8);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(&p_full[i], 8); mbar_init(&p_empty[i], 1); }
        abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base, AT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    gb_grid_wait();                                // q and the cache come from the kernels before
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * AT_BN, tmem_p = tmem_base + 3 * AT_BN;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&q_full, AT_TILE);
            tma_load_2d(q_s, &map_q, h * AT_HD, tok0, &q_full);
            tma_load_2d(q_s + AT_CHUNK, &map_q, h * AT_HD + 64, tok0, &q_full);
            for (int j = 0; j < n_blocks && !abort_flag; ++j) {
                const int s = j & 1;
                const uint32_t par = ((j >> 1) & 1) ^ 1;
                const int pages = min(2, pg_end - (pg_begin + 2 * j));          // the last block may hold one page
                if (!mbar_wait(&k_empty[s], par)) { atomicExch(p.status, 11); abort_flag = 1; break; }
                mbar_expect_tx(&k_full[s], pages * 2 * AT_PAGE_CHUNK);
                for (int pg = 0; pg < pages; ++pg) {
                    const int y = (trow[(pg_begin + 2 * j + pg) % p.ring_pages] * p.nkv + g) * GB_PAGE;
                    for (int c = 0; c < 2; ++c)
                        tma_load_2d(k_s + s * AT_TILE + c * AT_CHUNK + pg * AT_PAGE_CHUNK, &map_k, 64 * c, y, &k_full[s]);
                }
                if (!mbar_wait(&v_empty[s], par)) { atomicExch(p.status, 12); abort_flag = 1; break; }
                mbar_expect_tx(&v_full[s], pages * 2 * AT_PAGE_CHUNK);
                for (int pg = 0; pg < pages; ++pg) {
                    const int y = (trow[(pg_begin + 2 * j + pg) % p.ring_pages] * p.nkv + g) * GB_PAGE;
                    for (int c = 0; c < 2; ++c)
                        tma_load_2d(v_s + s * AT_TILE + c * AT_CHUNK + pg * AT_PAGE_CHUNK, &map_v, 64 * c, y, &v_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc_bf16(AT_BM, AT_BN);
            constexpr uint32_t idesc_pv = instr_desc_bf16_b_mn(AT_BM, AT_HD);
            bool ok = mbar_wait(&q_full, 0);
            if (!ok) { atomicExch(p.status, 13); abort_flag = 1; }
            auto issue_qk = [&](int j) {
                const int s = j & 1;
                const uint32_t par = (j >> 1) & 1;
                if (!mbar_wait(&k_full[s], par) || !mbar_wait(&s_empty[s], par ^ 1)) { atomicExch(p.status, 14); abort_flag = 1; ok = false; return; }
                tc_fence_after();
                const uint32_t qa = smem_u32(q_s), ka = smem_u32(k_s + s * AT_TILE);
#pragma unroll
                for (int k = 0; k < AT_HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * AT_CHUNK + (k & 3) * 32;
                    mma_f16(tmem_s + s * AT_BN, smem_desc_sw128(qa + off), smem_desc_sw128(ka + off), idesc_qk, k > 0 ? 1u : 0u);
                }
                mma_commit(&s_full[s]);
                mma_commit(&k_empty[s]);
            };
            if (ok && n_blocks > 0) issue_qk(0);
            for (int j = 0; j < n_blocks && ok && !abort_flag; ++j) {
                if (j + 1 < n_blocks) issue_qk(j + 1);            // runs under the softmax of block j
                if (!ok) break;
                const int s = j & 1;
                if (!mbar_wait(&v_full[s], (j >> 1) & 1) || !mbar_wait(&p_full[s], (j >> 1) & 1)) {
                    atomicExch(p.status, 15); abort_flag = 1; break;
                }
                tc_fence_after();
                const uint32_t va = smem_u32(v_s + s * AT_TILE);
#pragma unroll
                for (int k = 0; k < AT_BN / 16; ++k)
                    mma_f16_a_tmem(tmem_o, tmem_p + s * 64 + k * 8, smem_desc_sw128_mn(va + k * 2048, AT_CHUNK), idesc_pv,
                                   (j > 0 || k > 0) ? 1u : 0u);
                mma_commit(&p_empty[s]);              // this P buffer may be rewritten, and O holds this block's contribution
                mma_commit(&v_empty[s]);
            }
        }
    } else {
        // two warps per quarter of the rows: warps 2..5 take the first 64 keys of every block, warps 6..9 the
        // other 64; the two threads of a row agree on the row's maximum through shared memory
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;                       // query row = TMEM lane
        const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
        const int pq = r < rows ? pos_lo + r : -1;
        const int lo = p.window > 0 ? pq - p.window + 1 : 0;
        const float raise = 8.f / p.scale_log2;                  // the reference maximum follows only jumps beyond 2^8
        constexpr int HB = AT_BN / 2;                            // keys per thread and block
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory"); };
        for (int j = 0; j < n_blocks; ++j) {
            // after a wait has given up this warp only keeps its appointments with its partner (a named barrier
            // does not time out)
            if (!ok) { pair_sync(); continue; }
            const int s = j & 1;
            const int key0 = (pg_begin + 2 * j) * GB_PAGE + half * HB;
            if (!mbar_wait(&s_full[s], (j >> 1) & 1)) {
                if (lane == 0) atomicExch(p.status, 16);
                abort_flag = 1;
                ok = false;
                pair_sync();
                continue;
            }
            tc_fence_after();
            const uint32_t s_addr = tmem_s + s * AT_BN + half * HB + lane_addr;
            const bool need_mask = key0 + HB - 1 > pos_lo || p.window > 0 || r >= rows;
            float v[HB];
            tmem_ld64(s_addr, v);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[s]);               // S may be overwritten by the block after next
            float mx = -INFINITY;
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < HB; ++i) {
                    const int ka = key0 + i;
                    if (ka > pq || ka < lo) v[i] = -INFINITY;
                }
            }
            {
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains instead of one long one
#pragma unroll
                for (int i = 0; i < HB; i += 4) {
                    m4[0] = fmaxf(m4[0], v[i]); m4[1] = fmaxf(m4[1], v[i + 1]);
                    m4[2] = fmaxf(m4[2], v[i + 2]); m4[3] = fmaxf(m4[3], v[i + 3]);
                }
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            }
            mx_s[s][half][r] = mx;
            pair_sync();
            mx = fmaxf(mx, mx_s[s][half ^ 1][r]);
            // raise the reference when the maximum has run away from it (or there was none yet)
            float factor = 1.f;
            if (mx > -INFINITY && (m_ref == -INFINITY || mx > m_ref + raise)) {
                factor = m_ref == -INFINITY ? 0.f : exp2f((m_ref - mx) * p.scale_log2);
                m_ref = mx;
            }
            const float ms = m_ref == -INFINITY ? 0.f : m_ref * p.scale_log2;
            // two elements per instruction for the scaling and the sum; masked entries are -inf: 2^-inf is 0
            float add;
            {
                const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), ms2 = make_float2(-ms, -ms);
                float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
                for (int i = 0; i < HB; i += 2) {
                    float2 t = __ffma2_rn(make_float2(v[i], v[i + 1]), sc2, ms2);
                    t.x = ex2_approx(t.x);
                    t.y = ex2_approx(t.y);
                    v[i] = t.x;
                    v[i + 1] = t.y;
                    acc[(i >> 1) & 3] = __fadd2_rn(acc[(i >> 1) & 3], t);
                }
                const float2 a01 = __fadd2_rn(acc[0], acc[1]), a23 = __fadd2_rn(acc[2], acc[3]);
                add = (a01.x + a01.y) + (a23.x + a23.y);
            }
            if (j > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
                // O must hold every block before this one before its rows are rescaled
                if (!mbar_wait(&p_empty[s ^ 1], ((j - 1) >> 1) & 1)) { if (lane == 0) atomicExch(p.status, 17); abort_flag = 1; ok = false; continue; }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {                       // this thread's half of the row of O
                    float o[32];
                    tmem_ld32(tmem_o + lane_addr + half * 64 + 32 * c, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= factor;
                    tmem_st32(tmem_o + lane_addr + half * 64 + 32 * c, o);
                }
                tc_fence_before();
            }
            l = l * factor + add;
            // P as bf16 into this block's TMEM buffer, once the product of the block before last has read it
            if (!mbar_wait(&p_empty[s], ((j >> 1) & 1) ^ 1)) { if (lane == 0) atomicExch(p.status, 17); abort_flag = 1; ok = false; continue; }
            {
                uint32_t w[HB / 2];
#pragma unroll
                for (int i = 0; i < HB / 2; ++i) {
                    __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                    w[i] = *reinterpret_cast<uint32_t*>(&t);
                }
                tmem_st32_words(tmem_p + s * 64 + half * 32 + lane_addr, w);
                tc_fence_before();
            }
            if ((pg_begin + 2 * j) * GB_PAGE + AT_BN - 1 > valid_end) {
                // key row r of this block holds nothing meaningful if it lies beyond the sequence's end (never
                // written) or in a page this tile did not load: zero its values before they are multiplied
                // (each of the row's two threads zeroes one half of the head's dimensions)
                if (mbar_wait(&v_full[s], (j >> 1) & 1)) {
                    if ((pg_begin + 2 * j) * GB_PAGE + r > valid_end) {
                        uint4 z = make_uint4(0, 0, 0, 0);
                        for (int piece = 0; piece < 8; ++piece)
                            *reinterpret_cast<uint4*>(v_s + s * AT_TILE + half * AT_CHUNK + r * 128 + piece * 16) = z;
                    }
                    fence_proxy_async();                           // the patch is visible to the tensor core
                } else {
                    if (lane == 0) atomicExch(p.status, 18);
                    abort_flag = 1;
                    ok = false;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[s]);
        }
        // the last block's product has been added to O when its P buffer is free again
        if (ok && n_blocks > 0 && !mbar_wait(&p_empty[(n_blocks - 1) & 1], ((n_blocks - 1) >> 1) & 1)) {
            if (lane == 0) atomicExch(p.status, 19);
            ok = false;
        }
        tc_fence_after();
        l_s[half][r] = l;
        pair_sync();
        l += l_s[half ^ 1][r];
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = p.out + size_t(tok0 + r) * p.ldo + size_t(h) * AT_HD + half * 64;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
            float o[32];
            tmem_ld32(tmem_o + lane_addr + half * 64 + 32 * c, o);  // every lane takes part; rows beyond the tile are not stored
            if (r < rows && ok && n_blocks > 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    float t[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) t[e] = o[i + e] * inv;
                    *reinterpret_cast<uint4*>(dst + 32 * c + i) = pack8(t);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, AT_TMEM_COLS);
}

int* g_at_status_host = nullptr;
int* g_at_status_dev = nullptr;

}  // namespace

GB_API int gb_attention_prefill_tc_supported(int hd, int cache_dtype, int q_dtype) {
    return cache_dtype == GB_BF16 && q_dtype == GB_BF16 && hd == AT_HD;
}

GB_API int gb_attention_prefill_tc_tile() { return AT_BM; }

// q: bf16 [T, nh*128] (rotated) with pitch ldq; kcache, vcache: one run's pages [n_pages, nkv, 64, 128];
// tiles: (sequence row, first query) per 128 queries.  Same contract as gb_attention_prefill.
GB_API int gb_attention_prefill_tc(const void* q, long long ldq, void* out, long long ldo, int T, int nh, int nkv, int hd,
                                   const int* tiles, int n_tiles, const int* cu, const int* starts, const int* qlens,
                                   const int* table, int table_width, int ring_pages, const void* kcache,
                                   const void* vcache, long long n_pages, int window, float scale, cudaStream_t stream) {
    GB_REQUIRE(gb_attention_prefill_tc_supported(hd, GB_BF16, GB_BF16), "gb_attention_prefill_tc: head_dim %d is not 128", hd);
    GB_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "gb_attention_prefill_tc: bad head counts %d / %d", nh, nkv);
    GB_REQUIRE(n_tiles <= 65535, "gb_attention_prefill_tc: %d tiles of queries are too many for one launch", n_tiles);
    GB_REQUIRE(window >= 0 && ring_pages > 0 && table_width > 0 && n_pages > 0, "gb_attention_prefill_tc: bad cache geometry");
    GB_REQUIRE((ldo % 8) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0, "gb_attention_prefill_tc: misaligned output");
    if (n_tiles == 0) return 0;
    if (!g_at_status_host) {
        if (cudaHostAlloc(&g_at_status_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess)
            return gb_fail("gb_attention_prefill_tc: cannot allocate the status word");
        *g_at_status_host = 0;
        if (cudaHostGetDevicePointer(&g_at_status_dev, g_at_status_host, 0) != cudaSuccess)
            return gb_fail("gb_attention_prefill_tc: cannot map the status word");
    }
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM) != cudaSuccess)
            return gb_fail("gb_attention_prefill_tc: cannot get %d bytes of shared memory", AT_SMEM);
        configured = true;
    }
    CUtensorMap mq, mk, mv;
    if (tensor_map_bf16_2d(q, T, (long long)nh * hd, ldq, AT_BM, &mq)) return 1;
    if (tensor_map_bf16_2d(kcache, n_pages * nkv * GB_PAGE, hd, hd, GB_PAGE, &mk)) return 1;
    if (tensor_map_bf16_2d(vcache, n_pages * nkv * GB_PAGE, hd, hd, GB_PAGE, &mv)) return 1;
    AtParams p;
    p.out = (__nv_bfloat16*)out; p.tiles = tiles; p.cu = cu; p.starts = starts; p.qlens = qlens; p.table = table;
    p.status = g_at_status_dev; p.ldo = ldo; p.nh = nh; p.nkv = nkv; p.table_width = table_width;
    p.ring_pages = ring_pages; p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
    cudaError_t e = gb_launch(attention_prefill_tc_kernel, dim3(nh, n_tiles), dim3(AT_THREADS), AT_SMEM, stream, mq, mk, mv, p);
    if (e != cudaSuccess) return gb_fail("gb_attention_prefill_tc: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

// Non-zero when a bounded wait inside the kernel gave up since the last clear (read after a synchronise).
GB_API int gb_attention_tc_status() { return g_at_status_host ? *g_at_status_host : 0; }
GB_API int gb_attention_tc_status_clear() {
    if (g_at_status_host) *g_at_status_host = 0;
    return 0;
}
