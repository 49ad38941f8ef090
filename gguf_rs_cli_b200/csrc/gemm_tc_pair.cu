// The tensor-core product of gemm_tc.cu for steps of many tokens, with two CTAs on two SMs per output tile of
// 256 features x 256 tokens (tcgen05 cta_group::2).  Each CTA of the pair loads its 128 features of W and its
// 128 tokens of X for every block of K (32 KB a stage instead of the 48 KB a lone CTA needs for 128 x 256:
// a third less traffic from L2 into shared memory, and room for 6 stages), one thread of the even CTA (the
// leader) issues the MMAs for both, each CTA's TMEM gets its 128 features of the result, and each CTA's four
// epilogue warps finish those with the code the other kernel uses.
//
// Barriers: loads of both CTAs count their bytes on the leader's `full` barriers; the leader's MMA thread
// frees a stage in both CTAs and announces a finished accumulator to both with one multicast commit; the
// epilogue warps of both CTAs arrive on the leader's `acc_empty`.  Every wait is bounded (status word as in
// gemm_tc.cu); the cluster barriers at the start and at the end are reached by every thread on every path.
#include "gemm_tc.cuh"

using namespace sm100;

namespace {

constexpr int PBN = 256;                    // tokens per tile
constexpr int PHALF = PBN / 2;              // tokens a CTA loads
constexpr int PSTAGES = 6;
constexpr int PSTAGE_BYTES = A_BYTES + PHALF * BK * 2;         // per CTA
constexpr int POUT_CHUNK = 16 * BM * 2;      // a staged piece of the result: 16 tokens x 128 features of bf16
constexpr int POUT_RING = 4;                // pieces in flight to global memory
constexpr int PSMEM = PSTAGES * PSTAGE_BYTES + POUT_RING * POUT_CHUNK + 1024;
constexpr int PTMEM_COLS = 2 * PBN;         // two accumulators

struct PairUnit {
    int n0, t0;                             // first feature and first token of the 256 x 256 tile
};
// Tiles in the order of gemm_tc.cu's units: token tiles in groups of TILE_GROUP, inside a group feature tile
// by feature tile with the group's token tiles innermost.
__device__ __forceinline__ PairUnit pair_unit_of(int u, int feature_tiles, int token_tiles) {
    const int per_group = TILE_GROUP * feature_tiles;
    const int group = u / per_group, r = u - group * per_group;
    const int group_start = group * TILE_GROUP;
    const int group_size = min(TILE_GROUP, token_tiles - group_start);
    const int ft = r / group_size;
    PairUnit w;
    w.n0 = ft * (2 * BM);
    w.t0 = (group_start + (r - ft * group_size)) * PBN;
    return w;
}

template <bool STAGED>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                     const __grid_constant__ CUtensorMap map_x,
                                                                     const __grid_constant__ CUtensorMap map_o, TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* out_ring = ring + PSTAGES * PSTAGE_BYTES;
    __shared__ uint64_t full_bar[PSTAGES], empty_bar[PSTAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base;
    __shared__ float rstd_s[PBN];
    __shared__ float part_s[128];
    __shared__ float ssq_s[4][PBN];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();               // 0: leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int kb_total = (p.K + BK - 1) / BK;
    const int feature_tiles = (p.N + 2 * BM - 1) / (2 * BM);
    const int token_tiles = (p.T + PBN - 1) / PBN;
    const int n_units = feature_tiles * token_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 8); }
        fence_barrier_init();
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_x);
    }
    if (warp == 1) {
        tmem_alloc_pair(&tmem_base, PTMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();                             // both CTAs' barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_d = tmem_base;
    gb_grid_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer (both CTAs): this CTA's half of W's and of X's rows for every stage
            gb_grid_wait();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int u = pair; u < n_units && ok; u += n_pairs) {
                const PairUnit w = pair_unit_of(u, feature_tiles, token_tiles);
                for (int kb = 0; kb < kb_total; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { atomicExch(p.status, 1); ok = false; break; }
                    if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * PSTAGE_BYTES);
                    uint8_t* a = ring + stage * PSTAGE_BYTES;
                    tma_load_2d_pair(a, &map_w, kb * BK, w.n0 + int(rank) * BM, &full_bar[stage]);
                    tma_load_2d_pair(a + A_BYTES, &map_x, kb * BK, w.t0 + int(rank) * PHALF, &full_bar[stage]);
                    if (++stage == PSTAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issue (leader): 256 x 256 x 16 per instruction over the pair
            constexpr uint32_t idesc = instr_desc_bf16(2 * BM, PBN);
            int stage = 0, j = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int u = pair; u < n_units && ok; u += n_pairs, ++j) {
                const int buf = j & 1;
                if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1)) { atomicExch(p.status, 4); ok = false; break; }
                tc_fence_after();
                const uint32_t acc = tmem_d + buf * PBN;
                for (int kb = 0; kb < kb_total; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase)) { atomicExch(p.status, 2); ok = false; break; }
                    tc_fence_after();
                    uint32_t a = smem_u32(ring + stage * PSTAGE_BYTES);
                    uint32_t b = a + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_f16_pair(acc, smem_desc_sw128(a + k * UMMA_K * 2), smem_desc_sw128(b + k * UMMA_K * 2), idesc,
                                     (kb > 0 || k > 0) ? 1u : 0u);
                    mma_commit_pair(&empty_bar[stage]);
                    if (++stage == PSTAGES) { stage = 0; phase ^= 1; }
                }
                mma_commit_pair(&acc_full[buf]);
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue (both CTAs): this CTA's 128 features of the tile, warp w reads TMEM lanes 32*(w%4) .. +31
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        gb_grid_wait();
        int j = 0, piece = 0;
        for (int u = pair; u < n_units; u += n_pairs, ++j) {
            const PairUnit w = pair_unit_of(u, feature_tiles, token_tiles);
            const int buf = j & 1;
            const int n0 = w.n0 + int(rank) * BM;
            const int n = n0 + row;
            const int cols = min(PBN, p.T - w.t0);
            if (p.row_ssq) tc_token_scales<PBN>(p, w.t0, cols, row, rstd_s, part_s);
            const bool waited = mbar_wait(&acc_full[buf], (j >> 1) & 1);
            if (!waited) {
                if (lane == 0) atomicExch(p.status, 3);
                break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_d + (uint32_t(quarter * 32) << 16) + buf * PBN;
            float bias = 0.f;
            if (p.bias && n < p.N) bias = gb_load(p.bias, p.bias_dtype, n);
            if constexpr (STAGED) {
                // bf16 results: 16 tokens at a time into a ring of shared-memory pieces [token][feature], each
                // sent on its way by one TMA store (the scattered 2-byte stores from registers would take as
                // long as the tile's multiplications)
                for (int c0 = 0; c0 < cols; c0 += 16, ++piece) {
                    float v[16];
                    tmem_ld16(taddr + c0, v);
                    if (p.row_ssq) {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) v[jj] *= rstd_s[min(c0 + jj, PBN - 1)];
                    }
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out_ring + (piece % POUT_RING) * POUT_CHUNK);
                    if (threadIdx.x == 64) tma_store_source_free<POUT_RING - 1>();      // the piece's last store has read it
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (!p.swiglu) {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) dst[jj * BM + row] = __float2bfloat16_rn(v[jj] + bias);
                    } else {
                        // even rows are gate features, odd rows the matching up features (see tc_finish_chunk)
                        const bool odd = lane & 1;
                        float other[8];
#pragma unroll
                        for (int jj = 0; jj < 8; ++jj) other[jj] = __shfl_xor_sync(0xffffffffu, odd ? v[jj] : v[8 + jj], 1);
#pragma unroll
                        for (int jj = 0; jj < 8; ++jj) {
                            const float gte = odd ? other[jj] : v[jj], up = odd ? v[8 + jj] : other[jj];
                            dst[((odd ? 8 : 0) + jj) * (BM / 2) + (row >> 1)] = __float2bfloat16_rn(gte / (1.f + expf(-gte)) * up);
                        }
                    }
                    fence_proxy_async();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (threadIdx.x == 64 && waited)
                        tma_store_2d(&map_o, p.swiglu ? (n0 >> 1) : n0, w.t0 + c0, dst);
                }
            } else {
                for (int c0 = 0; c0 < cols; c0 += 16) {
                    float v[16];
                    tmem_ld16(taddr + c0, v);
                    tc_finish_chunk<PBN>(p, n0, w.t0, n, row, lane, quarter, bias, waited, c0, cols, v, rstd_s, ssq_s);
                }
                if (p.resid_x) tc_write_ssq<PBN>(p, n0, w.t0, row, 0, cols, ssq_s);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(&acc_empty[buf], 0);      // the leader may overwrite this accumulator
        }
        if (STAGED && threadIdx.x == 64) tma_store_done();
    }
    // nobody leaves while its partner may still read its shared memory or arrive on its barriers
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem_d, PTMEM_COLS);
}

}  // namespace

// How many pairs of CTAs of this kernel the device holds at once (0 if it cannot be asked).
static int pair_slots() {
    static int slots = -1;
    if (slots < 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2);
        cfg.blockDim = dim3(TC_THREADS);
        cfg.dynamicSmemBytes = PSMEM;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<true>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
        slots = n;
    }
    return slots;
}

int gemm_tc_pair_launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap* mo, const void* params,
                        cudaStream_t stream) {
    const TcParams& p = *static_cast<const TcParams*>(params);
    static int state = 0;                          // 1: ready, -1: refused
    if (state == 0) {
        state = cudaFuncSetAttribute(gemm_tc_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PSMEM) == cudaSuccess &&
                        cudaFuncSetAttribute(gemm_tc_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PSMEM) == cudaSuccess
                    ? 1 : -1;
        if (state < 0) cudaGetLastError();
    }
    if (state < 0) return gb_fail("gb_gemm_tc: cannot get %d bytes of shared memory", PSMEM);
    long long units = (long long)((p.N + 2 * BM - 1) / (2 * BM)) * ((p.T + PBN - 1) / PBN);
    long long slots = pair_slots() > 0 ? pair_slots() : p.sms / 2;     // pairs that can be resident at once
    long long rounds = (units + slots - 1) / slots;
    long long pairs = (units + rounds - 1) / rounds;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = PSMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gb_pdl_enabled() ? 2 : 1;
    if (mo)
        cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<true>, mw, mx, *mo, p);
    else
        cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<false>, mw, mx, mx, p);
    GB_LAUNCH_OK("gb_gemm_tc (pair)");
    return 0;
}
