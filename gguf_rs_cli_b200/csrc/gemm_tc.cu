// bf16 matrix product on the 5th-generation tensor cores:
//   out[t,n] = sum_k X[t,k] * W[n,k] (+ bias[n]),  f32 accumulation in TMEM.
//
// The weights are the M operand of tcgen05.mma (128 output features per tile), the
// tokens the N operand (16..256 per tile), so a decode step of a few tokens streams
// the weights through full 128-row instructions and a prompt of thousands of tokens
// uses 128x256 tiles; both operands are K-major, as the model folder stores W [out,in]
// (src/tensor/dequant.rs:258-259) and activations are [tokens, in].
//
// Persistent CTAs, no more than are resident at once, each with an equal share of all (tile, K block)
// pairs (gemm_tc.cuh).  6 warps: warp 0 issues TMA loads of
// 128-byte-swizzled [rows x 64] bf16 tiles into a ring of shared-memory stages, warp 1
// owns the TMEM allocation and issues the MMAs (one thread) into one of two accumulators,
// warps 2..5 read the other accumulator back (each its quarter of the 128 lanes) and
// store, so the epilogue of one unit runs under the main loop of the next.  Out-of-range rows
// and the K tail are zero-filled by TMA, so any T, any N, and any K that is a multiple
// of 8 (16-byte row pitch) work; other sizes are refused and the caller falls back to
// the CUDA-core kernel.
//
// A tile whose K blocks are spread over several CTAs (few tiles, as in decode, would leave SMs idle, and a
// number of tiles that is no multiple of the CTAs would leave some with twice the work) is merged by the last
// of them to arrive: each writes its partial tile to scratch memory and bumps the tile's counter, and the one
// that finds all others there adds the partial tiles in their fixed order and writes the result.  Nobody waits
// for anybody, the order of the sum does not depend on timing, and a CTA that is not the last leaves at once,
// which lets the CTAs of the next kernel on the stream take its place and ask for their weights early.
// (Merging a tile by all of its CTAs together, each adding up a share of the tokens once all had arrived,
// was built and measured: it needs every CTA to stay until the end, the next kernel starts later, and a decode
// step of the 8B shape at batch 8 took 3.74 ms instead of 3.34 ms.)
#include <mutex>
#include <unordered_map>

#include "gemm_tc.cuh"
#include "stamps.cuh"

using namespace sm100;

namespace {

// Barrier of the four epilogue warps that also tells every thread whether any of them raised `flag`.
__device__ __forceinline__ bool epilogue_any(bool flag) {
    uint32_t any;
    asm volatile(
        "{\n.reg .pred p, q;\n"
        "setp.ne.u32 q, %1, 0;\n"
        "barrier.cta.red.or.pred p, 1, 128, q;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(any)
        : "r"(uint32_t(flag))
        : "memory");
    return any != 0;
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// v[jj] = the sum over a shared tile's CTAs, in ascending order, of token c0 + jj of this thread's feature: S partial
// tiles x C tokens of loads in flight at a time (every round of loads costs a trip to L2, and the kernel after
// this one waits for it: few CTAs on a tile take more tokens per round).  base: the first CTA's first slot, at
// this thread's feature.
template <int BN, int S, int C>
__device__ __forceinline__ void sum_partials(const float* base, int first_which, int n_ctas, int c0, int cols, float (&v)[16]) {
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) v[jj] = 0.f;
#pragma unroll
    for (int j0 = 0; j0 < 16; j0 += C) {
        if (c0 + j0 >= cols) break;
        for (int s0 = 0; s0 < n_ctas; s0 += S) {
            float ld[S][C];
#pragma unroll
            for (int si = 0; si < S; ++si) {
                const int s = s0 + si;
                const float* part = base + (size_t(s) * 2 + (s == 0 ? first_which : 0)) * (BN * BM);
#pragma unroll
                for (int jj = 0; jj < C; ++jj)
                    ld[si][jj] = (s < n_ctas && c0 + j0 + jj < cols) ? __ldcg(part + (c0 + j0 + jj) * BM) : 0.f;
            }
#pragma unroll
            for (int si = 0; si < S; ++si)
#pragma unroll
                for (int jj = 0; jj < C; ++jj) v[j0 + jj] += ld[si][jj];
        }
    }
}

// Time stamps (builds with -DGB_STAMPS): slots of a CTA of the one product whose N and K were asked for.
// 0 entry, 1 the wait for the kernel in front is over, 2 the first operands are there, 3 the last MMA is committed,
// 4 the accumulator is seen complete, 5 partial sums stored and fenced, 6 counted (and the tile's other CTAs seen),
// 7 the sharers' sums of the first 16 tokens are there, 8 the tile (or this CTA's share) is finished, 9 exit.
#ifdef GB_STAMPS
__device__ long long* g_stamps = nullptr;
__device__ int g_stamps_n = 0, g_stamps_k = 0;
#define STAMP_IF(cond, k) if (cond) GB_STAMP_WRITE((p.N == g_stamps_n && p.K == g_stamps_k) ? g_stamps : nullptr, blockIdx.x, k)
#define STAMP_AFTER_IF(cond, k, val) if (cond) GB_STAMP_WRITE_AFTER((p.N == g_stamps_n && p.K == g_stamps_k) ? g_stamps : nullptr, blockIdx.x, k, val)
#else
#define STAMP_IF(cond, k)
#define STAMP_AFTER_IF(cond, k, val)
#endif

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, ctas_per_sm(BN)) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x, TcParams p) {
    using Cfg = TileCfg<BN>;
    constexpr bool SLICES = BN >= 32;        // every CTA of a shared tile finishes a share of its tokens (else the last one all)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full_bar[Cfg::STAGES], empty_bar[Cfg::STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base;
    __shared__ int last_flag;
    __shared__ float rstd_s[BN];            // per token of the tile: the deferred norm's scale
    __shared__ float part_s[128];
    __shared__ float ssq_s[4][BN];          // per epilogue warp and token: sum of squares of the new residual

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    STAMP_IF(threadIdx.x == 0, 0);
    const int kb_total = (p.K + BK - 1) / BK;
    const int token_tiles = (p.T + BN - 1) / BN;
    const int g_begin = cta_begin(blockIdx.x, p, kb_total), g_end = cta_begin(blockIdx.x + 1, p, kb_total);   // this CTA's share

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        fence_barrier_init();
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_x);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = tmem_base;
    gb_grid_launch_dependents();                    // the next kernel may begin its own prologue

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: TMA loads into the ring, unit after unit without a pause.  The weights do not
            // depend on the kernel before this one, so the first round of weight tiles is requested at
            // once; the activations only after that kernel has finished.
            int issued = 0;
            {
                UnitWalk walk(p, g_begin, g_end);
                Unit w;
                while (issued < Cfg::STAGES && walk.next(w, p, BN, token_tiles, kb_total))
                    for (int kb = w.kb_begin; kb < w.kb_end && issued < Cfg::STAGES; ++kb, ++issued) {
                        mbar_expect_tx(&full_bar[issued], Cfg::STAGE_BYTES);
                        tma_load_2d(ring + issued * Cfg::STAGE_BYTES, &map_w, kb * BK, w.n0, &full_bar[issued]);
                    }
            }
            const int pre = issued;
            gb_grid_wait();
            int item = 0, stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            UnitWalk walk(p, g_begin, g_end);
            Unit w;
            while (ok && walk.next(w, p, BN, token_tiles, kb_total)) {
                for (int kb = w.kb_begin; kb < w.kb_end; ++kb, ++item) {
                    uint8_t* a = ring + stage * Cfg::STAGE_BYTES;
                    if (item >= pre) {
                        if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { atomicExch(p.status, 1); ok = false; break; }
                        mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
                        tma_load_2d(a, &map_w, kb * BK, w.n0, &full_bar[stage]);
                    }
                    tma_load_2d(a + A_BYTES, &map_x, kb * BK, w.t0, &full_bar[stage]);
                    if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issue: two accumulators in TMEM, so that unit j+1 is multiplied while unit j is stored
            constexpr uint32_t idesc = instr_desc_bf16(BM, BN);
            int stage = 0, j = 0;
            uint32_t phase = 0;
            bool ok = true;
            UnitWalk walk(p, g_begin, g_end);
            Unit w;
            for (; ok && walk.next(w, p, BN, token_tiles, kb_total); ++j) {
                const int buf = j & 1;
                if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1)) { atomicExch(p.status, 4); ok = false; break; }
                tc_fence_after();
                const uint32_t acc = tmem_d + buf * BN;
                for (int kb = w.kb_begin; kb < w.kb_end; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase)) { atomicExch(p.status, 2); ok = false; break; }
                    STAMP_IF(j == 0 && kb == w.kb_begin, 2);
                    tc_fence_after();
                    uint32_t a = smem_u32(ring + stage * Cfg::STAGE_BYTES);
                    uint32_t b = a + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_f16(acc, smem_desc_sw128(a + k * UMMA_K * 2), smem_desc_sw128(b + k * UMMA_K * 2), idesc,
                                (kb > w.kb_begin || k > 0) ? 1u : 0u);
                    mma_commit(&empty_bar[stage]);      // the stage is free once these MMAs have read it
                    if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
                }
                mma_commit(&acc_full[buf]);             // this unit's accumulator is complete
                STAMP_IF(true, 3);
            }
        }
    } else {
        // ---- epilogue: 4 warps, warp w reads TMEM lanes 32*(w%4) .. +31.  The code that finishes 16 tokens of
        // a tile exists once, for tiles of the CTA's own and for shared ones (every SM runs this code from a cold
        // instruction cache after another kernel: its size is time).
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;        // feature within the tile = TMEM lane
        int j = 0;
        gb_grid_wait();                             // before anything is read or written that the kernel before touches
        STAMP_IF(threadIdx.x == 64, 1);
        UnitWalk walk(p, g_begin, g_end);
        Unit w;
        for (; walk.next(w, p, BN, token_tiles, kb_total); ++j) {
            const int buf = j & 1;
            const int n = w.n0 + row;
            const int cols = min(BN, p.T - w.t0);       // valid tokens of this tile
            const bool whole = w.kb_begin == 0 && w.kb_end == kb_total;
            // What the kernel before left for this tile is fetched while the products still run: the sums of
            // squares behind the tokens' scales and, in the 16-token kernel, this thread's row of the residual
            // stream (each a trip to L2 that the kernel after this one would otherwise wait for).
            float bias = 0.f;
            if (p.bias && n < p.N) bias = gb_load(p.bias, p.bias_dtype, n);
            if (p.row_ssq) tc_token_scales<BN>(p, w.t0, cols, row, rstd_s, part_s);
            float x_early[16];
            if (BN == 16 && p.resid_x) {
#pragma unroll
                for (int c = 0; c < 16; ++c)
                    x_early[c] = (n < p.N && c < cols) ? __ldcg(p.resid_x + size_t(w.t0 + c) * p.ld_x + n) : 0.f;
            }
            // A tile that several CTAs work on: which they are.  The tile's first CTA may have begun before the
            // tile (its partial sums then lie in its second slot); all others begin inside it.
            int first_cta = 0, n_ctas = 1, first_which = 0, me = 0;
            if (!whole) {
                tile_ctas(w.tile, p, kb_total, first_cta, n_ctas);
                first_which = cta_begin(first_cta, p, kb_total) < w.tile * kb_total ? 1 : 0;
                me = int(blockIdx.x) - first_cta;
            }
            // all four warps go on, or none: a warp that left alone would miss the others' barriers
            if (epilogue_any(!mbar_wait(&acc_full[buf], (j >> 1) & 1))) {
                if (threadIdx.x == 64) atomicExch(p.status, 3);
                break;
            }
            tc_fence_after();
            STAMP_IF(threadIdx.x == 64, 4);
            const uint32_t taddr = tmem_d + (uint32_t(quarter * 32) << 16) + buf * BN;
            bool finish = true;                          // does this CTA write the tile's result?
            bool sliced = false;                         // ... or a share of it, as every CTA of the tile does
            int c_lo = 0, c_hi = cols;                   // the tokens of the tile that it finishes
            if (!whole) {
                // this CTA's share of the tile: the partial sums go to scratch memory
                // (a partial tile lies token by token, each token's 128 features side by side: a warp's stores and loads
                // of one token are one 128-byte line; feature by feature with 16-byte accesses was measured: slower)
                float* mine = p.scratch + (size_t(blockIdx.x) * 2 + (me == 0 ? first_which : 0)) * (BN * BM) + row;
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    if (c0 >= cols) break;               // uniform over the warp
                    float v[16];
                    tmem_ld16(taddr + c0, v);
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj)
                        if (c0 + jj < cols) __stcg(mine + (c0 + jj) * BM, v[jj]);
                }
                tc_fence_before();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);     // the accumulator may be overwritten
                // The partial sums are at L2 before the counter counts this CTA (stores that bypass L1, a fence by
                // every thread that stored, a barrier, then the atomic).  The CTA that sees all others counted reads
                // their sums from L2 (__ldcg), after a barrier behind the atomic: nothing of it can run ahead, and it
                // needs no fence of its own.  The barrier in front of the next atomic also keeps last_flag from being
                // written before every thread has read it.
                __threadfence();
                epilogue_sync();
                STAMP_IF(threadIdx.x == 64, 5);
                if (SLICES && p.cut == CUT_PER_TILE) {
                    // Wide tiles: every CTA of the tile stays until all have counted themselves (a bounded wait) and
                    // finishes its own share of the tile's tokens, where the last CTA alone would spend 3 to 4 us on
                    // every 16 of them.  All CTAs of the kernel are resident when any of them waits (cut_for gives it
                    // no more CTAs than fit the device; the kernel behind starts only when all of this one have).
                    if (threadIdx.x == 64) {
                        atomicAdd(&p.counters[w.tile], 1);
                        int seen = 0;
                        uint64_t start = 0;
                        for (uint32_t i = 0; (seen = ld_acquire_gpu(&p.counters[w.tile])) < n_ctas; ++i) {
                            __nanosleep(40);
                            if ((i & 255) == 255) {          // gives up after about two seconds
                                const uint64_t now = global_timer_ns();
                                if (start == 0) start = now;
                                else if (now - start > WAIT_NS) break;
                            }
                        }
                        last_flag = seen >= n_ctas;
                    }
                    epilogue_sync();
                    if (!last_flag) {                      // uniform: the flag is shared
                        if (threadIdx.x == 64) atomicExch(p.status, 5);
                        break;
                    }
                    STAMP_IF(threadIdx.x == 64, 6);
                    c_lo = me * cols / n_ctas;
                    c_hi = (me + 1) * cols / n_ctas;
                    finish = c_lo < c_hi;
                    sliced = true;
                } else {
                    if (threadIdx.x == 64) last_flag = atomicAdd(&p.counters[w.tile], 1) == n_ctas - 1;
                    epilogue_sync();
                    STAMP_IF(threadIdx.x == 64, 6);
                    finish = last_flag != 0;
                }
            }
            if (finish) {
                for (int c0 = c_lo & ~15; c0 < c_hi; c0 += 16) {
                    float v[16], xv[16];
                    bool have_x = false;
                    if (whole) {
                        tmem_ld16(taddr + c0, v);
                    } else {
                        // the last CTA of a shared tile: its rows of the residual stream are asked for with the
                        // partial sums, not after them (one trip to L2 instead of two for every 16 tokens; tiles of 16
                        // tokens have them already, and with tiles of 32 it measured slower: 5.17 against 5.07 ms
                        // a step at 64 tokens, where tiles of 64 gain 0.05 of 5.9 ms at 128 tokens)
                        if (BN >= 64 && p.resid_x) {
#pragma unroll
                            for (int jj = 0; jj < 16; ++jj)
                                xv[jj] = (n < p.N && c0 + jj >= c_lo && c0 + jj < c_hi)
                                             ? __ldcg(p.resid_x + size_t(w.t0 + c0 + jj) * p.ld_x + n) : 0.f;
                            have_x = true;
                        }
                        const float* base = p.scratch + size_t(first_cta) * 2 * (BN * BM) + row;
                        if (n_ctas <= 4) sum_partials<BN, 4, 16>(base, first_which, n_ctas, c0, c_hi, v);
                        else sum_partials<BN, 8, 8>(base, first_which, n_ctas, c0, c_hi, v);
                        STAMP_AFTER_IF(threadIdx.x == 64 && c0 == (c_lo & ~15), 7, v[0] + v[7]);
                    }
                    if constexpr (BN == 16)
                        tc_finish_chunk<BN>(p, w.n0, w.t0, n, row, lane, quarter, bias, true, c0, c_hi, v, rstd_s, ssq_s,
                                            p.resid_x ? x_early : nullptr, c_lo);
                    else
                        tc_finish_chunk<BN>(p, w.n0, w.t0, n, row, lane, quarter, bias, true, c0, c_hi, v, rstd_s, ssq_s,
                                            have_x ? xv : nullptr, c_lo);
                }
                if (p.resid_x) tc_write_ssq<BN>(p, w.n0, w.t0, row, c_lo, c_hi, ssq_s);
                STAMP_IF(threadIdx.x == 64, 8);
                if (!whole && !sliced && threadIdx.x == 64) p.counters[w.tile] = 0;       // ready for the next launch
            }
            if (sliced) {
                // the last of the tile's CTAs to have read the others' sums puts the counter back for the next launch
                epilogue_sync();
                if (threadIdx.x == 64 && atomicAdd(&p.counters[w.tile], 1) == 2 * n_ctas - 1) p.counters[w.tile] = 0;
            }
            if (whole) {
                tc_fence_before();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);     // all of this warp's TMEM loads are done
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    STAMP_IF(threadIdx.x == 0, 9);
    if (warp == 1) tmem_dealloc(tmem_d, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    long long rows, cols, ld;
    int box_rows, box_cols;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && box_cols == o.box_cols;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        for (long long v : {k.rows, k.cols, k.ld, (long long)k.box_rows, (long long)k.box_cols}) h = h * 1000003u ^ std::hash<long long>()(v);
        return h;
    }
};

// Tensor map of a row-major bf16 matrix [rows, cols] with pitch ld: box [box_rows x 64] with the 128-byte swizzle
// (operands), or, with box_cols given, [box_rows x box_cols] without a swizzle (tiles stored from shared memory).
int tensor_map_2d(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out,
                  int box_cols = 0) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, ld, box_rows, box_cols};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return gb_fail("gb_gemm_tc: the driver gives no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
    cuuint32_t box[2] = {cuuint32_t(box_cols ? box_cols : BK), cuuint32_t(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return gb_fail("gb_gemm_tc: cuTensorMapEncodeTiled failed with code %d", int(r));
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

int* g_status_host = nullptr;
int* g_status_dev = nullptr;

int ensure_status() {
    if (g_status_host) return 0;
    if (cudaHostAlloc(&g_status_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess)
        return gb_fail("gb_gemm_tc: cannot allocate the status word");
    *g_status_host = 0;
    if (cudaHostGetDevicePointer(&g_status_dev, g_status_host, 0) != cudaSuccess)
        return gb_fail("gb_gemm_tc: cannot map the status word");
    return 0;
}

constexpr int MAX_DEVICES = 64;

template <int BN>
int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, cudaStream_t stream, bool pdl = true) {
    using Cfg = TileCfg<BN>;
    // the shared-memory limit is an attribute of the function on each device; the first launch of a tile width
    // on a device sets it
    static bool configured[MAX_DEVICES] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return gb_fail("gb_gemm_tc: no usable current device");
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess)
            return gb_fail("gb_gemm_tc: cannot get %d bytes of shared memory", Cfg::SMEM);
        configured[dev] = true;
    }
    gb_launch_opt(gemm_tc_kernel<BN>, dim3(p.n_ctas), dim3(TC_THREADS), Cfg::SMEM, stream, pdl, mw, mx, p);
    GB_LAUNCH_OK("gb_gemm_tc");
    return 0;
}

}  // namespace

// Tokens per tile for T tokens.
GB_API int gb_gemm_tc_tile(int T) { return T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256; }

// Tuning aids (process-wide; the defaults are what every caller wants).
static int g_tile_override = 0;       // > 0: tokens per tile for every product
GB_API int gb_gemm_tc_set_tile(int bn) { g_tile_override = bn; return 0; }
static int g_pair = 1;                // 0: never two SMs per tile
GB_API int gb_gemm_tc_set_pair(int on) { g_pair = on; return 0; }
static int g_mode = 0;                // 0: by the rule below, 1: whole tiles only, 2: equal shares of K blocks where tiles are not shared out per tile, 3: equal shares always
GB_API int gb_gemm_tc_set_mode(int mode) { g_mode = mode; return 0; }

// The same with the number of output features known: a few hundred tokens with few features would
// give 256-token tiles for less than half of the SMs, so they take 128-token tiles.
static int tile_for(int T, int N, int sms) {
    if (g_tile_override > 0) return g_tile_override;
    int bn = gb_gemm_tc_tile(T);
    const long long ft = (N + BM - 1) / BM;
    if (bn == 256 && 2 * ft * ((T + 255) / 256) <= sms) bn = 128;
    // (A few dozen tokens used to take two half-size token tiles where there are fewer feature tiles than SMs,
    // because the one CTA that finished a shared tile read all its partial tiles.  Since every CTA of a tile of
    // 32 tokens or more finishes a share of it, whole-width tiles are faster: batch 24 to 64 of the 8B shape
    // 3.87 / 3.94 / 4.60 / 4.71 instead of 4.07 / 4.10 / 4.79 / 4.84 ms a step.)
    // a few hundred tokens: tiles of 64 tokens, two CTAs per SM, as long as all of them fit the device at once
    // (a CTA with a wide tile streams its operands no faster; measured at 128 to 768 tokens)
    if (bn >= 128 && (T <= 128 || ft * ((T + 63) / 64) <= 2LL * sms)) bn = 64;
    return bn;
}

// How a product of these sizes is cut (gemm_tc.cuh): tile width, CTAs, and whether CTAs share tiles.
struct TcCut {
    int bn, n_ctas, cut, per_tile, extra, kb;
    long long tiles, scratch_floats;
    void fill(TcParams& p) const {
        p.n_ctas = n_ctas; p.tiles = int(tiles); p.cut = cut; p.per_tile = per_tile; p.extra = extra;
        p.total_its = int(tiles * kb); p.its_each = p.total_its / n_ctas; p.its_rest = p.total_its % n_ctas;
    }
};
static TcCut cut_for(int T, int N, int K, int sms, bool may_share, int n_counters) {
    TcCut c;
    c.bn = tile_for(T, N, sms);
    c.tiles = (long long)((N + BM - 1) / BM) * ((T + c.bn - 1) / c.bn);
    c.kb = (K + BK - 1) / BK;
    const long long slots = (long long)ctas_per_sm(c.bn) * (sms > 0 ? sms : 1);        // CTAs that are resident at once
    c.cut = CUT_WHOLE;
    c.per_tile = c.extra = 0;
    c.scratch_floats = 0;
    c.n_ctas = 1;
    if (c.tiles == 0) return c;              // no tokens: nothing is launched
    // whole tiles: every CTA the same number of tiles, or one less
    const long long rounds = (c.tiles + slots - 1) / slots;
    c.n_ctas = int((c.tiles + rounds - 1) / rounds);
    // Few tiles: several CTAs per tile, each with a part of the tile's K blocks, at least 4 K blocks a CTA (8 where K
    // is long: 4096 x 4096 at 8 to 16 tokens took 9.3 instead of 9.9 us) and no more than 16 CTAs on one tile (the
    // last of them reads all their partial tiles).  Tiles of 256 tokens go to the kernel that pairs two SMs.
    const bool pair = c.bn == 256 && g_pair;
    if (!may_share || pair || c.tiles > n_counters || g_mode == 1) return c;
    long long n = c.tiles * c.kb / (c.kb >= 64 ? 8 : 4);
    n = n > slots ? slots : n < 1 ? 1 : n;
    if (n > 16 * c.tiles) n = 16 * c.tiles;
    if (n >= 2 * c.tiles && g_mode != 3) {
        // what is left over when every tile has the same number of CTAs goes to the first tiles, one CTA each,
        // unless that would leave the shares more than 6% apart
        long long q = n / c.tiles, r = n % c.tiles;
        if (100 * r > 6 * q * c.tiles) r = 0;
        c.n_ctas = int(q * c.tiles + r);
        c.cut = CUT_PER_TILE;
        c.per_tile = int(q);
        c.extra = int(r);
        c.scratch_floats = 2LL * c.n_ctas * c.bn * BM;
    } else if (g_mode >= 2 && n != c.tiles && c.tiles % n != 0) {
        // Equal shares of all K blocks wherever they fall (a tuning aid: measured on the 8B shape, gate and up at
        // batch 8 with 224 tiles on 296 CTAs, the two merges per CTA cost more than the idle SMs: 3.60 instead of
        // 3.43 ms a step).
        c.n_ctas = int(n);
        c.cut = CUT_EVEN;
        c.scratch_floats = 2LL * n * c.bn * BM;
    }
    return c;
}

// CTAs that a product of these sizes runs on, on a device with `sms` SMs, when it may use scratch memory.
GB_API int gb_gemm_tc_ctas(int T, int N, int K, int sms) { return cut_for(T, N, K, sms, true, 1 << 30).n_ctas; }

// Floats of scratch a launch with these sizes needs (0 when no tile is shared between CTAs).
GB_API long long gb_gemm_tc_scratch_floats(int T, int N, int K, int sms) {
    return cut_for(T, N, K, sms, true, 1 << 30).scratch_floats;
}

// Whether the tensor-core kernel takes these operands (bf16, 16-byte aligned, pitches multiples of 8).
GB_API int gb_gemm_tc_supported(const void* X, long long ldx, const void* W, long long ldw, int K) {
    return K >= 8 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(W) & 15) == 0;
}

// X: bf16 [T, K] pitch ldx; W: bf16 [N, K] pitch ldw; out: bf16 or f32 [T, N] pitch ldo; bias optional.
// W must not be written by the kernel that runs before this one on the stream: the first tiles of W are
// requested before that kernel has finished (the engine's W are constant weights).
// scratch: gb_gemm_tc_scratch_floats(...) floats; counters: at least as many zeroed ints as tiles
// (the kernel leaves them zero).  Both may be null: every CTA then takes whole tiles.
// swiglu_features > 0: W is [2*64*ceil(F/64), K], row 2f being gate row f and row 2f+1 up row f (zero
// rows pad the last tile), F = swiglu_features, and
// out[t,f] = silu(gate_f) * up_f has F columns (src/model/llama.rs:399-401 in the product's epilogue).
static int gemm_tc_impl(const void* X, long long ldx, const void* W, long long ldw, const void* bias, int bias_dtype,
                        void* out, int out_dtype, long long ldo, int T, int N, int K, float* scratch, int* counters,
                        int n_counters, int sms, int swiglu_features, const float* row_ssq, int ssq_parts, int norm_size,
                        float eps, float* resid_x, void* resid_xb, float* ssq_out, long long ld_x, cudaStream_t stream);

GB_API int gb_gemm_tc(const void* X, long long ldx, const void* W, long long ldw, const void* bias, int bias_dtype,
                      void* out, int out_dtype, long long ldo, int T, int N, int K, float* scratch, int* counters,
                      int n_counters, int sms, int swiglu_features, cudaStream_t stream) {
    return gemm_tc_impl(X, ldx, W, ldw, bias, bias_dtype, out, out_dtype, ldo, T, N, K, scratch, counters, n_counters, sms,
                        swiglu_features, nullptr, 0, 0, 0.f, nullptr, nullptr, nullptr, 0, stream);
}

// The same product with a deferred RMS norm on its input and/or a residual epilogue:
//  - row_ssq [ssq_parts, T] (f32): X holds rows that were not normalised (the norm's weight is folded into W);
//    every result is scaled by 1 / sqrt(sum_i row_ssq[i][t] / norm_size + eps) before bias and activation;
//  - resid_x [T, N] f32 with pitch ld_x: instead of writing `out`, x += result (+ bias) in place, resid_xb (bf16,
//    same pitch) gets the rounded copy, and ssq_out [ceil(N/128), T] the sums of squares of the new x over each
//    tile of 128 features: the row_ssq of the product that reads xb next.
GB_API int gb_gemm_tc_fused(const void* X, long long ldx, const void* W, long long ldw, const void* bias, int bias_dtype,
                            void* out, int out_dtype, long long ldo, int T, int N, int K, float* scratch, int* counters,
                            int n_counters, int sms, int swiglu_features, const float* row_ssq, int ssq_parts,
                            int norm_size, float eps, float* resid_x, void* resid_xb, float* ssq_out, long long ld_x,
                            cudaStream_t stream) {
    GB_REQUIRE(!row_ssq || (ssq_parts > 0 && norm_size > 0 && eps > 0.f), "gb_gemm_tc_fused: bad norm parameters");
    GB_REQUIRE(!resid_x || (resid_xb && ssq_out && ld_x >= N && !swiglu_features), "gb_gemm_tc_fused: bad residual parameters");
    return gemm_tc_impl(X, ldx, W, ldw, bias, bias_dtype, out, out_dtype, ldo, T, N, K, scratch, counters, n_counters, sms,
                        swiglu_features, row_ssq, ssq_parts, norm_size, eps, resid_x, resid_xb, ssq_out, ld_x, stream);
}

static int gemm_tc_impl(const void* X, long long ldx, const void* W, long long ldw, const void* bias, int bias_dtype,
                        void* out, int out_dtype, long long ldo, int T, int N, int K, float* scratch, int* counters,
                        int n_counters, int sms, int swiglu_features, const float* row_ssq, int ssq_parts, int norm_size,
                        float eps, float* resid_x, void* resid_xb, float* ssq_out, long long ld_x, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(out_dtype) && (!bias || gb_is_dtype(bias_dtype)), "gb_gemm_tc: bad dtype");
    GB_REQUIRE(T >= 0 && N > 0 && K > 0, "gb_gemm_tc: bad sizes T=%d N=%d K=%d", T, N, K);
    GB_REQUIRE(swiglu_features >= 0 && (resid_x || ldo >= (swiglu_features ? swiglu_features : N)), "gb_gemm_tc: output pitch %lld too small", ldo);
    GB_REQUIRE(!swiglu_features || (N == 128 * ((swiglu_features + 63) / 64) && !bias),
               "gb_gemm_tc: a gated product of %d features needs %d interleaved rows and no bias, got %d", swiglu_features,
               128 * ((swiglu_features + 63) / 64), N);
    GB_REQUIRE(gb_gemm_tc_supported(X, ldx, W, ldw, K),
               "gb_gemm_tc: K=%d and the row pitches (%lld, %lld) must be multiples of 8 and the operands 16-byte aligned",
               K, ldx, ldw);
    if (T == 0) return 0;
    if (ensure_status()) return 1;
    const TcCut cut = cut_for(T, N, K, sms, scratch && counters, n_counters);
    GB_REQUIRE(cut.tiles * cut.kb < (1LL << 31) - (1 << 20), "gb_gemm_tc: T=%d N=%d K=%d is more work than the kernel numbers", T, N, K);
    const int bn = cut.bn;
    TcParams p;
    p.out = out; p.bias = bias; p.scratch = scratch; p.counters = counters; p.status = g_status_dev;
    p.ldo = ldo; p.out_dtype = out_dtype; p.bias_dtype = bias_dtype; p.T = T; p.N = N; p.K = K;
    p.swiglu = swiglu_features > 0; p.N_out = swiglu_features; p.sms = sms;
    cut.fill(p);
    p.row_ssq = row_ssq; p.ssq_parts = ssq_parts; p.norm_size = norm_size; p.eps = eps;
    p.resid_x = resid_x; p.resid_xb = (__nv_bfloat16*)resid_xb; p.ssq_out = ssq_out; p.ld_x = ld_x;
    CUtensorMap mw, mx;
    if (tensor_map_2d(W, N, K, ldw, BM, &mw)) return 1;
    if (bn == 256 && g_pair && cut.cut == CUT_WHOLE) {
        // many tokens: two SMs per 256 x 256 tile, each loading 128 tokens of X per stage; bf16 results leave
        // through shared memory and TMA stores of [16 tokens x 128 features] (64 features after SwiGLU)
        if (tensor_map_2d(X, T, K, ldx, 128, &mx)) return 1;
        CUtensorMap mo;
        const bool staged = !resid_x && out_dtype == GB_BF16 && ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
        if (staged && tensor_map_2d(out, T, swiglu_features ? swiglu_features : N, ldo, 16, &mo, swiglu_features ? 64 : 128)) return 1;
        return gemm_tc_pair_launch(mw, mx, staged ? &mo : nullptr, &p, stream);
    }
    if (tensor_map_2d(X, T, K, ldx, bn, &mx)) return 1;
    switch (bn) {
        case 16: return launch_tc<16>(mw, mx, p, stream);
        case 32: return launch_tc<32>(mw, mx, p, stream);
        case 64: return launch_tc<64>(mw, mx, p, stream);
        case 128: return launch_tc<128>(mw, mx, p, stream);
        default: return launch_tc<256>(mw, mx, p, stream);
    }
}

// Non-zero when a bounded wait inside a tensor-core kernel gave up since the last clear
// (1: a load stage never came free, 2: a load never arrived, 3/4: an accumulator never completed or never came free).
// Read after synchronising the stream.
// Builds with -DGB_STAMPS: the CTAs of every product of N features over K write their time stamps to buf
// (16 64-bit slots a CTA; null: none do).
GB_API int gb_gemm_tc_set_stamps(long long* buf, int n, int k) {
#ifdef GB_STAMPS
    if (cudaMemcpyToSymbol(g_stamps_n, &n, sizeof(n)) != cudaSuccess || cudaMemcpyToSymbol(g_stamps_k, &k, sizeof(k)) != cudaSuccess ||
        cudaMemcpyToSymbol(g_stamps, &buf, sizeof(buf)) != cudaSuccess)
        return gb_fail("gb_gemm_tc_set_stamps: cannot set the buffer");
    return 0;
#else
    (void)buf; (void)n; (void)k;
    return gb_fail("gb_gemm_tc_set_stamps: this library was built without -DGB_STAMPS");
#endif
}
GB_API int gb_tc_status() { return g_status_host ? *g_status_host : 0; }
GB_API int gb_tc_status_clear() {
    if (g_status_host) *g_status_host = 0;
    return 0;
}

// ------------------------------------------------------------ no-allocation entry point
// See gemm_tc_noalloc.h.  The scratch of the K split lives in the library image.  In host code
// the names below are host-side stand-ins, not device addresses; the device addresses are
// looked up once per device with cudaGetSymbolAddress and handed to the kernel.
#include "gemm_tc_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[GB_NOALLOC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_noalloc_counters[GB_NOALLOC_COUNTERS];
static __device__ __align__(256) int g_noalloc_status;

namespace {

constexpr int NOALLOC_MAX_DEVICES = 64;
struct NoallocDevice {
    bool ready;
    float* scratch;
    int* counters;
    int* status;
    int sms;
};
NoallocDevice g_noalloc_dev[NOALLOC_MAX_DEVICES];      // zero-initialised; one slot per device ordinal
std::mutex g_noalloc_mu;

// Address look-up for the current device, once.
int noalloc_setup(int dev, NoallocDevice** out) {
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return gb_fail("gb_gemm_tc_noalloc: device ordinal %d is out of range", dev);
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    NoallocDevice& d = g_noalloc_dev[dev];
    if (!d.ready) {
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.scratch), g_noalloc_scratch);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.counters), g_noalloc_counters);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status), g_noalloc_status);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess)
            return gb_fail("gb_gemm_tc_noalloc: cannot find the built-in scratch on device %d: %s", dev, cudaGetErrorString(e));
        d.ready = true;
    }
    *out = &d;
    return 0;
}

// A tensor map built on the caller's stack, without the cache that gb_gemm_tc keeps on the heap.
int encode_map_2d(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return gb_fail("gb_gemm_tc_noalloc: the driver gives no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
    cuuint32_t box[2] = {cuuint32_t(BK), cuuint32_t(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return gb_fail("gb_gemm_tc_noalloc: cuTensorMapEncodeTiled failed with code %d", int(r));
    return 0;
}

}  // namespace

GB_API int gb_gemm_tc_noalloc(const void* X, long long ldx, const void* W, long long ldw, const void* bias,
                              int bias_dtype, void* out, int out_dtype, long long ldo, int T, int N, int K,
                              cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(out_dtype) && (!bias || gb_is_dtype(bias_dtype)), "gb_gemm_tc_noalloc: bad dtype");
    GB_REQUIRE(T >= 0 && N > 0 && K > 0 && ldo >= N, "gb_gemm_tc_noalloc: bad sizes T=%d N=%d K=%d ldo=%lld", T, N, K, ldo);
    GB_REQUIRE(gb_gemm_tc_supported(X, ldx, W, ldw, K),
               "gb_gemm_tc_noalloc: K=%d and the row pitches (%lld, %lld) must be multiples of 8 and the operands 16-byte "
               "aligned", K, ldx, ldw);
    if (T == 0) return 0;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return gb_fail("gb_gemm_tc_noalloc: no current device");
    NoallocDevice* d = nullptr;
    if (noalloc_setup(dev, &d)) return 1;
    // the same cut of the work as gb_gemm_tc makes; tiles that CTAs share need scratch memory and counters
    const TcCut cut = cut_for(T, N, K, d->sms, true, 1 << 30);
    GB_REQUIRE(cut.tiles * cut.kb < (1LL << 31) - (1 << 20), "gb_gemm_tc_noalloc: T=%d N=%d K=%d is more work than the kernel numbers", T, N, K);
    const int bn = cut.bn;
    if (cut.cut != CUT_WHOLE) {
        GB_REQUIRE(cut.scratch_floats <= GB_NOALLOC_SCRATCH_FLOATS && cut.tiles <= GB_NOALLOC_COUNTERS,
                   "gb_gemm_tc_noalloc: T=%d N=%d K=%d runs on %d CTAs that share %lld tiles and needs %lld floats of scratch; "
                   "the built-in scratch holds %d floats and %d tiles (use gb_gemm_tc with memory of your own)",
                   T, N, K, cut.n_ctas, cut.tiles, cut.scratch_floats, GB_NOALLOC_SCRATCH_FLOATS, GB_NOALLOC_COUNTERS);
        // the arrival counters must start at zero whatever an earlier call left behind
        if (cudaMemsetAsync(d->counters, 0, sizeof(int) * size_t(cut.tiles), stream) != cudaSuccess)
            return gb_fail("gb_gemm_tc_noalloc: cannot clear the counters");
    }
    TcParams p;
    p.out = out; p.bias = bias; p.scratch = d->scratch; p.counters = d->counters; p.status = d->status;
    p.ldo = ldo; p.out_dtype = out_dtype; p.bias_dtype = bias_dtype; p.T = T; p.N = N; p.K = K;
    p.swiglu = 0; p.N_out = 0; p.sms = d->sms;
    cut.fill(p);
    p.row_ssq = nullptr; p.ssq_parts = 0; p.norm_size = 0; p.eps = 0.f;
    p.resid_x = nullptr; p.resid_xb = nullptr; p.ssq_out = nullptr; p.ld_x = 0;
    CUtensorMap mw, mx;
    if (encode_map_2d(W, N, K, ldw, BM, &mw)) return 1;
    if (encode_map_2d(X, T, K, ldx, bn, &mx)) return 1;
    // An ordinary launch, not a programmatic dependent one: the kernel asks for its first tiles of W before it
    // waits for the kernel in front of it, which is right for constant weights but not for a caller whose W may
    // be the output of the call before.
    switch (bn) {
        case 16: return launch_tc<16>(mw, mx, p, stream, false);
        case 32: return launch_tc<32>(mw, mx, p, stream, false);
        case 64: return launch_tc<64>(mw, mx, p, stream, false);
        case 128: return launch_tc<128>(mw, mx, p, stream, false);
        default: return launch_tc<256>(mw, mx, p, stream, false);
    }
}

GB_API int gb_gemm_tc_noalloc_status(void) {
    int dev = -1, value = 0, zero = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES || !g_noalloc_dev[dev].ready) return 0;
    if (cudaMemcpy(&value, g_noalloc_dev[dev].status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (value) cudaMemcpy(g_noalloc_dev[dev].status, &zero, sizeof(int), cudaMemcpyHostToDevice);
    return value;
}
