// Attention for prompts on the 5th-generation tensor cores (head sizes 64 and 128): the same
// arithmetic as attention_prefill.cu and the generic kernel (src/model/llama.rs:374-394),
// with both products of flash attention issued as tcgen05.mma and their results in TMEM.
//
// A CTA owns 256 consecutive queries of one sequence and one head as two tiles of 128 and walks
// the keys in blocks of 128 (two cache pages) that both tiles share.  18 warps:
//   warp 0  TMA: both Q tiles once, then K and V pages into two-stage rings (128-byte swizzle);
//   warp 1  one thread issues, tile by tile, S = Q K^T (M128 N128, K = head size) into the tile's TMEM
//           buffer and, when the tile's probabilities are ready, O += P V (P read from TMEM,
//           V from shared memory N-contiguous, as the cache stores it) into the tile's
//           output accumulator, which stays in TMEM for the whole tile.  While one tile's
//           warps work on their softmax the tensor core serves the other tile;
//   warps 2-9 and 10-17  one tile each, two threads per query row (its TMEM lane), each with 64
//           of a block's 128 keys: maximum (agreed between the two through shared memory), sum and
//           probabilities in 32-bit; P goes back as bf16 into the first half of the columns S came from.
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

constexpr int AT_BM = 128, AT_BN = 128;
constexpr int AT_PAIR = 2 * AT_BM;             // queries per CTA
constexpr int AT_THREADS = 576;                // TMA, MMA and two tiles of eight softmax warps
constexpr int AT_CHUNK = 128 * 128;            // bytes of a [128 rows x 64 columns] bf16 tile
constexpr int AT_PAGE_CHUNK = 64 * 128;        // bytes of a [64 rows x 64 columns] piece of a page
constexpr int AT_TMEM_COLS = 512;              // per tile: S (128 columns; P in its first 64) and O (head size)
template <int HD> struct AtCfg {
    static constexpr int CHUNKS = HD / 64;               // [128 x 64] pieces of a [128 x HD] tile
    static constexpr int TILE = CHUNKS * AT_CHUNK;       // 32 KB at head size 128
    static constexpr int SMEM = 6 * TILE + 1024;         // Q x2, K x2, V x2 (+ alignment slack)
};

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

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1) attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                             const __grid_constant__ CUtensorMap map_k,
                                                                             const __grid_constant__ CUtensorMap map_v,
                                                                             AtParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int AT_TILE = AtCfg<HD>::TILE, CHUNKS = AtCfg<HD>::CHUNKS;
    uint8_t* q_s = base;                         // 2 tiles
    uint8_t* k_s = base + 2 * AT_TILE;           // 2 stages
    uint8_t* v_s = base + 4 * AT_TILE;           // 2 stages
    __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], pv_done[2];
    __shared__ uint32_t tmem_base;
    __shared__ volatile int abort_flag;
    __shared__ float mx_s[2][2][2][AT_BM], l_s[2][2][AT_BM];      // exchanged between the two threads of a query row

    gb_grid_launch_dependents();
    // the list holds tiles of 128 queries; this kernel takes them two at a time, from the even ones
    const int b = p.tiles[2 * blockIdx.y], q0 = p.tiles[2 * blockIdx.y + 1];
    if (q0 % AT_PAIR != 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x, g = h / (p.nh / p.nkv);
    const int start = p.starts[b], qlen = p.qlens[b], tok0 = p.cu[b] + q0;
    const int last_pos = start + qlen - 1;
    // per tile: its rows, the positions of its first and last query, and its blocks [first, end) in the grid
    // of 128-key blocks that starts at the page of the earliest key the first tile may see
    int rows[2], pos_lo[2], blk_first[2], blk_end[2];
    const int lo0 = p.window > 0 ? max(0, start + q0 - p.window + 1) : 0;
    const int pg_base = lo0 >> GB_PAGE_SHIFT;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        rows[t] = max(0, min(AT_BM, qlen - q0 - t * AT_BM));
        pos_lo[t] = start + q0 + t * AT_BM;
        const int lo = p.window > 0 ? max(0, pos_lo[t] - p.window + 1) : 0;
        blk_first[t] = rows[t] > 0 ? ((lo >> GB_PAGE_SHIFT) - pg_base) / 2 : 0;
        blk_end[t] = rows[t] > 0 ? (((pos_lo[t] + rows[t] - 1) >> GB_PAGE_SHIFT) - pg_base) / 2 + 1 : 0;
    }
    const int n_blocks = max(blk_end[0], blk_end[1]);
    const int pos_hi = start + q0 + rows[0] + rows[1] - 1;                 // the CTA's last query
    const int pg_end = (pos_hi >> GB_PAGE_SHIFT) + 1;
    const int valid_end = min(last_pos, pg_end * GB_PAGE - 1);   // last key position that was both written and loaded
    const int* trow = p.table + size_t(b) * p.table_width;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 8); mbar_init(&pv_done[i], 1);
        }
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
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * AT_BN;     // + tile * 128 each

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&q_full, 2 * AT_TILE);
            for (int t = 0; t < 2; ++t)
                for (int c = 0; c < CHUNKS; ++c)
                    tma_load_2d(q_s + t * AT_TILE + c * AT_CHUNK, &map_q, h * HD + 64 * c, tok0 + t * AT_BM, &q_full);
            for (int j = 0; j < n_blocks && !abort_flag; ++j) {
                const int s = j & 1;
                const uint32_t par = ((j >> 1) & 1) ^ 1;
                const int pages = min(2, pg_end - (pg_base + 2 * j));          // the last block may hold one page
                if (!mbar_wait(&k_empty[s], par)) { atomicExch(p.status, 11); abort_flag = 1; break; }
                mbar_expect_tx(&k_full[s], pages * CHUNKS * AT_PAGE_CHUNK);
                for (int pg = 0; pg < pages; ++pg) {
                    const int y = (trow[(pg_base + 2 * j + pg) % p.ring_pages] * p.nkv + g) * GB_PAGE;
                    for (int c = 0; c < CHUNKS; ++c)
                        tma_load_2d(k_s + s * AT_TILE + c * AT_CHUNK + pg * AT_PAGE_CHUNK, &map_k, 64 * c, y, &k_full[s]);
                }
                if (!mbar_wait(&v_empty[s], par)) { atomicExch(p.status, 12); abort_flag = 1; break; }
                mbar_expect_tx(&v_full[s], pages * CHUNKS * AT_PAGE_CHUNK);
                for (int pg = 0; pg < pages; ++pg) {
                    const int y = (trow[(pg_base + 2 * j + pg) % p.ring_pages] * p.nkv + g) * GB_PAGE;
                    for (int c = 0; c < CHUNKS; ++c)
                        tma_load_2d(v_s + s * AT_TILE + c * AT_CHUNK + pg * AT_PAGE_CHUNK, &map_v, 64 * c, y, &v_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc_bf16(AT_BM, AT_BN);
            constexpr uint32_t idesc_pv = instr_desc_bf16_b_mn(AT_BM, HD);
            bool ok = mbar_wait(&q_full, 0);
            if (!ok) { atomicExch(p.status, 13); abort_flag = 1; }
            auto active = [&](int t, int j) { return j >= blk_first[t] && j < blk_end[t]; };
            // S of tile t for block j; it overwrites the tile's S and P of the block before, whose product was
            // issued earlier by this thread
            auto issue_qk = [&](int t, int j) {
                const int s = j & 1;
                if (!mbar_wait(&k_full[s], (j >> 1) & 1)) { atomicExch(p.status, 14); abort_flag = 1; ok = false; return; }
                tc_fence_after();
                const uint32_t qa = smem_u32(q_s + t * AT_TILE), ka = smem_u32(k_s + s * AT_TILE);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * AT_CHUNK + (k & 3) * 32;
                    mma_f16(tmem_s + t * AT_BN, smem_desc_sw128(qa + off), smem_desc_sw128(ka + off), idesc_qk, k > 0 ? 1u : 0u);
                }
                mma_commit(&s_full[t]);
            };
            int done[2] = {0, 0};                              // blocks multiplied into O per tile
            for (int t = 0; t < 2 && ok; ++t)
                if (active(t, 0)) issue_qk(t, 0);
            if (ok && n_blocks > 0) mma_commit(&k_empty[0]);
            for (int j = 0; j < n_blocks && ok && !abort_flag; ++j) {
                const int s = j & 1;
                for (int t = 0; t < 2 && ok; ++t) {
                    if (active(t, j)) {
                        if (!mbar_wait(&v_full[s], (j >> 1) & 1) || !mbar_wait(&p_full[t], done[t] & 1)) {
                            atomicExch(p.status, 15); abort_flag = 1; ok = false; break;
                        }
                        tc_fence_after();
                        const uint32_t va = smem_u32(v_s + s * AT_TILE);
#pragma unroll
                        for (int k = 0; k < AT_BN / 16; ++k)
                            mma_f16_a_tmem(tmem_o + t * HD, tmem_s + t * AT_BN + k * 8, smem_desc_sw128_mn(va + k * 2048, AT_CHUNK),
                                           idesc_pv, (done[t] > 0 || k > 0) ? 1u : 0u);
                        mma_commit(&pv_done[t]);              // O of the tile holds this block
                        ++done[t];
                    }
                    if (j + 1 < n_blocks && active(t, j + 1)) issue_qk(t, j + 1);     // runs under the other tile's softmax
                }
                if (!ok) break;
                mma_commit(&v_empty[s]);
                if (j + 1 < n_blocks) mma_commit(&k_empty[(j + 1) & 1]);
            }
        }
    } else {
        // eight warps per tile: two threads per query row, each with 64 of a block's 128 keys (warps 2..5 and
        // 10..13: the first 64; 6..9 and 14..17: the other 64); the two agree on the row's maximum through
        // shared memory.  A thread that has given up on a wait keeps its appointments with its partner (a named
        // barrier does not time out).
        const int t = (warp - 2) >> 3;                           // the tile of this warp
        const int half = ((warp - 2) >> 2) & 1;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                       // query row of the tile = TMEM lane
        const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
        const uint32_t s_addr = tmem_s + t * AT_BN + lane_addr, o_addr = tmem_o + t * HD + half * (HD / 2) + lane_addr;
        const int pq = r < rows[t] ? pos_lo[t] + r : -1;
        const int lo = p.window > 0 ? pq - p.window + 1 : 0;
        const float raise = 8.f / p.scale_log2;                  // the reference maximum follows only jumps beyond 2^8
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + t * 4 + quarter) : "memory"); };
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        int c = 0;                                               // blocks done by this tile
        for (int j = blk_first[t]; j < blk_end[t]; ++j, ++c) {
            if (!ok) { pair_sync(); continue; }
            const int s = j & 1;
            const int key0 = (pg_base + 2 * j) * GB_PAGE + half * 64;
            if (!mbar_wait(&s_full[t], c & 1)) {
                if (lane == 0) atomicExch(p.status, 16);
                abort_flag = 1;
                ok = false;
                pair_sync();
                continue;
            }
            tc_fence_after();
            float v[64];
            tmem_ld64(s_addr + 64 * half, v);
            if (key0 + 63 > pos_lo[t] || p.window > 0 || r >= rows[t]) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int ka = key0 + i;
                    if (ka > pq || ka < lo) v[i] = -INFINITY;
                }
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains instead of one long one
#pragma unroll
            for (int i = 0; i < 64; i += 4) {
                m4[0] = fmaxf(m4[0], v[i]); m4[1] = fmaxf(m4[1], v[i + 1]);
                m4[2] = fmaxf(m4[2], v[i + 2]); m4[3] = fmaxf(m4[3], v[i + 3]);
            }
            float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            mx_s[t][c & 1][half][r] = mx;
            pair_sync();                                         // both halves of S are in registers from here on
            mx = fmaxf(mx, mx_s[t][c & 1][half ^ 1][r]);
            // raise the reference when the maximum has run away from it (or there was none yet)
            float factor = 1.f;
            if (mx > -INFINITY && (m_ref == -INFINITY || mx > m_ref + raise)) {
                factor = m_ref == -INFINITY ? 0.f : exp2f((m_ref - mx) * p.scale_log2);
                m_ref = mx;
            }
            if (c > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
                // O must hold every block before this one before its rows are rescaled (this thread's half of them)
                if (!mbar_wait(&pv_done[t], (c - 1) & 1)) { if (lane == 0) atomicExch(p.status, 17); abort_flag = 1; ok = false; continue; }
                tc_fence_after();
#pragma unroll 1
                for (int cc = 0; cc < CHUNKS; ++cc) {
                    float o[32];
                    tmem_ld32(o_addr + 32 * cc, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= factor;
                    tmem_st32(o_addr + 32 * cc, o);
                }
                tc_fence_before();
            }
            // probabilities (two elements per instruction for the scaling and the sum; masked entries are -inf:
            // 2^-inf is 0), as bf16 over the first half of the columns S came from: this thread's 64 keys into
            // columns 32 * half .. + 31 (the partner has read them, see the barrier above)
            const float ms = m_ref == -INFINITY ? 0.f : m_ref * p.scale_log2;
            const float2 ms2 = make_float2(-ms, -ms);
            float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            uint32_t w[32];
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                float2 e = __ffma2_rn(make_float2(v[i], v[i + 1]), sc2, ms2);
                e.x = ex2_approx(e.x);
                e.y = ex2_approx(e.y);
                acc[(i >> 1) & 3] = __fadd2_rn(acc[(i >> 1) & 3], e);
                __nv_bfloat162 pk = __floats2bfloat162_rn(e.x, e.y);
                w[i >> 1] = *reinterpret_cast<uint32_t*>(&pk);
            }
            const float2 a01 = __fadd2_rn(acc[0], acc[1]), a23 = __fadd2_rn(acc[2], acc[3]);
            l = l * factor + ((a01.x + a01.y) + (a23.x + a23.y));
            tmem_st32_words(s_addr + 32 * half, w);
            tc_fence_before();
            if ((pg_base + 2 * j) * GB_PAGE + AT_BN - 1 > valid_end) {
                // key row r of this block holds nothing meaningful if it lies beyond the sequence's end (never
                // written) or in a page this CTA did not load: zero its values before they are multiplied (both
                // tiles do so before their own product of this block; each of a row's two threads one half)
                if (mbar_wait(&v_full[s], (j >> 1) & 1)) {
                    if ((pg_base + 2 * j) * GB_PAGE + r > valid_end) {
                        uint4 z = make_uint4(0, 0, 0, 0);
                        for (int i = 0; i < HD / 16; ++i) {
                            const int piece = half * (HD / 16) + i;          // 16-byte pieces of the row, eight per chunk
                            *reinterpret_cast<uint4*>(v_s + s * AT_TILE + (piece >> 3) * AT_CHUNK + r * 128 + (piece & 7) * 16) = z;
                        }
                    }
                    fence_proxy_async();                           // the patch is visible to the tensor core
                } else {
                    if (lane == 0) atomicExch(p.status, 18);
                    abort_flag = 1;
                    ok = false;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[t]);
        }
        // the tile's last product has been added to O
        if (ok && c > 0 && !mbar_wait(&pv_done[t], (c - 1) & 1)) { if (lane == 0) atomicExch(p.status, 19); ok = false; }
        tc_fence_after();
        l_s[t][half][r] = l;
        pair_sync();
        l += l_s[t][half ^ 1][r];
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = p.out + size_t(tok0 + t * AT_BM + r) * p.ldo + size_t(h) * HD + half * (HD / 2);
        if (c > 0) {
#pragma unroll 1
            for (int cc = 0; cc < CHUNKS; ++cc) {
                float o[32];
                tmem_ld32(o_addr + 32 * cc, o);                    // every lane takes part; rows beyond the tile are not stored
                if (r < rows[t] && ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float tt[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) tt[e] = o[i + e] * inv;
                        *reinterpret_cast<uint4*>(dst + 32 * cc + i) = pack8(tt);
                    }
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
    return cache_dtype == GB_BF16 && q_dtype == GB_BF16 && (hd == 64 || hd == 128);
}

GB_API int gb_attention_prefill_tc_tile() { return AT_BM; }

// q: bf16 [T, nh*hd] (rotated) with pitch ldq; kcache, vcache: one run's pages [n_pages, nkv, 64, hd];
// tiles: (sequence row, first query) per 128 queries.  Same contract as gb_attention_prefill.
GB_API int gb_attention_prefill_tc(const void* q, long long ldq, void* out, long long ldo, int T, int nh, int nkv, int hd,
                                   const int* tiles, int n_tiles, const int* cu, const int* starts, const int* qlens,
                                   const int* table, int table_width, int ring_pages, const void* kcache,
                                   const void* vcache, long long n_pages, int window, float scale, cudaStream_t stream) {
    GB_REQUIRE(gb_attention_prefill_tc_supported(hd, GB_BF16, GB_BF16), "gb_attention_prefill_tc: head_dim %d is neither 64 nor 128", hd);
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
        if (cudaFuncSetAttribute(attention_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, AtCfg<64>::SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(attention_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, AtCfg<128>::SMEM) != cudaSuccess)
            return gb_fail("gb_attention_prefill_tc: cannot get %d bytes of shared memory", AtCfg<128>::SMEM);
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
    cudaError_t e = hd == 64 ? gb_launch(attention_prefill_tc_kernel<64>, dim3(nh, n_tiles), dim3(AT_THREADS), AtCfg<64>::SMEM, stream, mq, mk, mv, p)
                             : gb_launch(attention_prefill_tc_kernel<128>, dim3(nh, n_tiles), dim3(AT_THREADS), AtCfg<128>::SMEM, stream, mq, mk, mv, p);
    if (e != cudaSuccess) return gb_fail("gb_attention_prefill_tc: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

// Non-zero when a bounded wait inside the kernel gave up since the last clear (read after a synchronise).
GB_API int gb_attention_tc_status() { return g_at_status_host ? *g_at_status_host : 0; }
GB_API int gb_attention_tc_status_clear() {
    if (g_at_status_host) *g_at_status_host = 0;
    return 0;
}
