// What the tensor-core product kernels share: tile sizes, the parameter block, the numbering of the units
// of work, and the last steps of an output tile (the deferred norm's scale per token, bias, the gated
// activation, the residual update).  gemm_tc.cu: one CTA per tile; gemm_tc_pair.cu: two CTAs (two SMs) per tile.
#pragma once
#include "common.cuh"
#include "sm100.cuh"

namespace {

constexpr int BM = 128;       // output features per tile (MMA M)
constexpr int BK = 64;        // K per stage: one 128-byte swizzled row of bf16
constexpr int UMMA_K = 16;
constexpr int TC_THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;

template <int BN> struct TileCfg {
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // small token tiles keep the ring near 100 KB so that two CTAs share an SM (more tiles in flight,
    // no idle half wave when there are between one and two tiles per SM)
    static constexpr int STAGES = BN >= 256 ? 4 : BN >= 128 ? 6 : BN >= 64 ? 4 : BN >= 32 ? 5 : 6;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;     // + slack to align the ring to 1024 bytes
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;      // two accumulators
};

// CTAs of the one-CTA kernel that share an SM (by shared memory; the kernel's launch bounds say the same).
__host__ __device__ constexpr int ctas_per_sm(int bn) { return bn <= 64 ? 2 : 1; }

struct TcParams {
    void* out;
    const void* bias;
    float* scratch;       // [2 * CTAs][BN][128] partial sums of the tiles that several CTAs share
    int* counters;        // [tiles], zero between launches
    int* status;          // set non-zero when a bounded wait gave up
    long long ldo;
    int out_dtype, bias_dtype;
    int T, N, K;
    int swiglu, N_out;    // swiglu: W's rows alternate gate, up; out has N_out features
    int sms;
    // how the work is cut (see Unit): CTAs, tiles, and the rule that gives each CTA its share
    int n_ctas, tiles, cut;   // cut: CUT_WHOLE, CUT_EVEN or CUT_PER_TILE
    int per_tile, extra;      // CUT_PER_TILE: every tile has per_tile CTAs, the first `extra` tiles one more
    int total_its;            // tiles * K blocks (the entry point refuses sizes beyond 2^31)
    int its_each, its_rest;   // total_its / n_ctas and total_its % n_ctas
    // deferred RMS norm of the input: X holds the un-normalised rows (the norm's weight is folded into W), and
    // the result is scaled per token by 1 / sqrt(sum_i row_ssq[i][t] / norm_size + eps)
    const float* row_ssq;
    int ssq_parts, norm_size;
    float eps;
    // residual epilogue: x[t,n] += result (32-bit, in place), xb = bf16(x), and the sum over this tile's 128
    // features of x^2 goes to ssq_out[feature tile][t] for the norm that comes next
    float* resid_x;
    __nv_bfloat16* resid_xb;
    float* ssq_out;
    long long ld_x;
};

// The work of a product is the sequence of all (tile, K block) pairs, tile after tile: tiles * kb_total
// iterations, cut into one contiguous share per CTA, with no more CTAs than are resident at once.  A CTA's
// share is cut into units at tile borders.  A unit that covers all of its tile's K blocks is finished by its
// CTA alone; a tile that several CTAs share is merged by all of them (gemm_tc.cu).  Three rules:
//   CUT_WHOLE     whole tiles only, CTA c taking every CTAs-th tile from tile c on (no shared tiles, no scratch)
//   CUT_EVEN      CTA c takes the iterations [c * total / CTAs, (c + 1) * total / CTAs): every CTA streams the
//                 same number of operand bytes whatever the sizes are; a share may end inside one tile and
//                 begin inside another
//   CUT_PER_TILE  fewer tiles than CTAs: every tile gets CTAs / tiles CTAs of its own (the first CTAs % tiles
//                 tiles one more), each an equal part of the tile's K blocks; no share crosses a tile border
// Tiles are numbered so that the CTAs running at one time share operands in L2: token tiles in groups of
// TILE_GROUP, inside a group feature tile by feature tile with the group's token tiles innermost (many
// tokens: the group's activations stay in L2 while the weights stream; few tokens: one group, feature-major
// as the weights lie in memory).
enum { CUT_WHOLE = 0, CUT_EVEN = 1, CUT_PER_TILE = 2 };
constexpr int TILE_GROUP = 16;
struct Unit {
    int tile, n0, t0, kb_begin, kb_end;
};
__device__ __forceinline__ void tile_origin(int tile, const TcParams& p, int BN, int token_tiles, int& n0, int& t0) {
    const int feature_tiles = (p.N + BM - 1) / BM;
    const int per_group = TILE_GROUP * feature_tiles;
    const int group = tile / per_group, r = tile - group * per_group;
    const int group_start = group * TILE_GROUP;
    const int group_size = min(TILE_GROUP, token_tiles - group_start);
    const int ft = r / group_size;
    n0 = ft * BM;
    t0 = (group_start + (r - ft * group_size)) * BN;
}
// CUT_PER_TILE: the tile of CTA c and the first CTA and number of CTAs of tile t.
__device__ __forceinline__ int per_tile_first(int t, const TcParams& p) { return t * p.per_tile + min(t, p.extra); }
__device__ __forceinline__ int per_tile_count(int t, const TcParams& p) { return p.per_tile + (t < p.extra ? 1 : 0); }
__device__ __forceinline__ int per_tile_of(int c, const TcParams& p) {
    const int wide = p.extra * (p.per_tile + 1);
    return c < wide ? c / (p.per_tile + 1) : p.extra + (c - wide) / p.per_tile;
}
// First iteration of CTA c (c = n_ctas gives the end of all work).  32-bit arithmetic throughout: a 64-bit
// division is a subroutine of a hundred instructions, inlined wherever it stands, and this code runs once per
// CTA from a cold instruction cache.
__device__ __forceinline__ int cta_begin(int c, const TcParams& p, int kb_total) {
    if (p.cut == CUT_WHOLE) return 0;       // not used: see UnitWalk
    if (p.cut == CUT_EVEN) return c * p.its_each + c * p.its_rest / p.n_ctas;      // = c * total / CTAs
    if (c >= p.n_ctas) return p.total_its;
    const int t = per_tile_of(c, p);
    return t * kb_total + (c - per_tile_first(t, p)) * kb_total / per_tile_count(t, p);
}
// The CTA whose share holds iteration g under CUT_EVEN: an estimate in floating point, put right by comparing.
__device__ __forceinline__ int cta_holding(int g, const TcParams& p, int kb_total) {
    int c = int((float(g) + 0.5f) * float(p.n_ctas) / float(p.total_its));
    c = min(max(c, 0), p.n_ctas - 1);
    while (c + 1 < p.n_ctas && cta_begin(c + 1, p, kb_total) <= g) ++c;
    while (c > 0 && cta_begin(c, p, kb_total) > g) --c;
    return c;
}
// The first CTA and the number of CTAs of a shared tile (CUT_EVEN and CUT_PER_TILE).
__device__ __forceinline__ void tile_ctas(int tile, const TcParams& p, int kb_total, int& first, int& count) {
    if (p.cut == CUT_PER_TILE) {
        first = per_tile_first(tile, p);
        count = per_tile_count(tile, p);
        return;
    }
    first = cta_holding(tile * kb_total, p, kb_total);
    count = cta_holding(tile * kb_total + kb_total - 1, p, kb_total) - first + 1;
}
// The units of this CTA, in the order it works on them.  With whole tiles CTA c takes the tiles c, c + CTAs,
// c + 2 CTAs, ...: the CTAs that run at one time then work on neighbouring tiles, whose operands they share in L2
// (CTA c taking tiles 2c and 2c + 1 instead made gate and up at 128 tokens read W twice from memory: 85 instead
// of 60 us).  Otherwise the units are the pieces of the CTA's share of the iterations.
struct UnitWalk {
    int g, g_end, tile, whole;
    __device__ __forceinline__ UnitWalk(const TcParams& p, int begin, int end)
        : g(begin), g_end(end), tile(blockIdx.x), whole(p.cut == CUT_WHOLE) {}
    __device__ __forceinline__ bool next(Unit& u, const TcParams& p, int BN, int token_tiles, int kb_total) {
        if (whole) {
            if (tile >= p.tiles) return false;
            u.tile = tile;
            u.kb_begin = 0;
            u.kb_end = kb_total;
            tile += p.n_ctas;
        } else {
            if (g >= g_end) return false;
            u.tile = g / kb_total;
            u.kb_begin = g - u.tile * kb_total;
            const int left = g_end - g;
            u.kb_end = left < kb_total - u.kb_begin ? u.kb_begin + left : kb_total;
            g += u.kb_end - u.kb_begin;
        }
        if (token_tiles == 1) {             // few tokens: tile t is feature tile t
            u.n0 = u.tile * BM;
            u.t0 = 0;
        } else {
            tile_origin(u.tile, p, BN, token_tiles, u.n0, u.t0);
        }
        return true;
    }
};

// The scale of each token of a tile under a deferred norm (the splits of one tile all compute the same
// numbers): the 128 epilogue threads share the loads, GROUPS threads per token each summing every GROUPS-th
// part with several loads in flight, then one of them adds the groups' sums in order.  rstd_s[c] is valid for
// c < cols afterwards.
template <int BN>
__device__ __forceinline__ void tc_token_scales(const TcParams& p, int t0, int cols, int row, float* rstd_s, float* part_s) {
    constexpr int SLOTS = BN < 128 ? BN : 128, GROUPS = 128 / SLOTS;
    const int slot = row % SLOTS, grp = row / SLOTS;
    for (int c0 = 0; c0 < BN; c0 += SLOTS) {
        const int c = c0 + slot;
        float ss = 0.f;
        if (c < cols) {
            const float* src = p.row_ssq + t0 + c;
            for (int i = grp; i < p.ssq_parts; i += 4 * GROUPS) {
                float ld[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    ld[e] = i + e * GROUPS < p.ssq_parts ? __ldcg(src + size_t(i + e * GROUPS) * p.T) : 0.f;
#pragma unroll
                for (int e = 0; e < 4; ++e) ss += ld[e];
            }
        }
        part_s[grp * SLOTS + slot] = ss;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (grp == 0 && c < cols) {
            float tot = 0.f;
#pragma unroll
            for (int gi = 0; gi < GROUPS; ++gi) tot += part_s[gi * SLOTS + slot];
            rstd_s[c] = 1.f / sqrtf(tot / float(p.norm_size) + p.eps);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
    }
}

// The sums of v[0] .. v[15], each over the warp's 32 lanes, in 16 shuffles instead of 80: at every step a lane keeps
// half of its values and hands the other half to the lane that keeps those.  Bit for bit gb_warp_sum's sums (the same
// pairs are added in the same order).  Lane L ends with the sum of the value whose index has bits 3..0 = L's bits 4..1.
__device__ __forceinline__ float tc_warp_sum16(const float (&v)[16], int lane) {
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4, h2 = lane & 2;
    float a[8], b[4], c[2];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = (h16 ? v[i + 8] : v[i]) + __shfl_xor_sync(0xffffffffu, h16 ? v[i] : v[i + 8], 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) b[i] = (h8 ? a[i + 4] : a[i]) + __shfl_xor_sync(0xffffffffu, h8 ? a[i] : a[i + 4], 8);
#pragma unroll
    for (int i = 0; i < 2; ++i) c[i] = (h4 ? b[i + 2] : b[i]) + __shfl_xor_sync(0xffffffffu, h4 ? b[i] : b[i + 2], 4);
    float d = (h2 ? c[1] : c[0]) + __shfl_xor_sync(0xffffffffu, h2 ? c[0] : c[1], 2);
    d += __shfl_xor_sync(0xffffffffu, d, 1);
    return d;
}

// The last steps for 16 columns (tokens c0 .. c0+15 of the tile, those from c_lo on and below c_end being the
// caller's to finish) of this thread's feature row n = n0 + row: v[jj] holds the finished sum of column c0 + jj.
// x_early: the 16 values of the residual stream at these places if the caller has read them already, else null.
template <int BN>
__device__ __forceinline__ void tc_finish_chunk(const TcParams& p, int n0, int t0, int n, int row, int lane, int quarter,
                                                float bias, bool waited, int c0, int c_end, float (&v)[16],
                                                const float* rstd_s, float (*ssq_s)[BN], const float* x_early = nullptr,
                                                int c_lo = 0) {
    auto mine = [&](int c) { return c >= c_lo && c < c_end; };
    if (p.row_ssq) {
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) v[jj] *= rstd_s[min(c0 + jj, BN - 1)];
    }
    if (p.resid_x) {
        // x += result; the bf16 copy and the tile's share of sum(x^2) per token for the next norm.
        // All of x is read before anything is written, so that the loads are in flight together.
        float xv[16];
#pragma unroll
        for (int jj = 0; jj < 16; ++jj)
            xv[jj] = x_early ? x_early[jj]
                             : (n < p.N && mine(c0 + jj)) ? __ldcg(p.resid_x + size_t(t0 + c0 + jj) * p.ld_x + n) : 0.f;
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
            float sq = 0.f;
            if (n < p.N && mine(c0 + jj)) {
                const size_t at = size_t(t0 + c0 + jj) * p.ld_x + n;
                const float xn = xv[jj] + v[jj] + bias;
                p.resid_x[at] = xn;
                p.resid_xb[at] = __float2bfloat16_rn(xn);
                sq = xn * xn;
            }
            v[jj] = sq;
        }
        const float sq = tc_warp_sum16(v, lane);
        const int jj = ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
        if ((lane & 1) == 0 && mine(c0 + jj)) ssq_s[quarter][c0 + jj] = sq;
    } else if (!p.swiglu) {
        if (n < p.N && waited) {
#pragma unroll
            for (int jj = 0; jj < 16; ++jj)
                if (mine(c0 + jj))
                    gb_store(p.out, p.out_dtype, size_t(t0 + c0 + jj) * p.ldo + n, v[jj] + bias);
        }
    } else {
        // even rows of the tile are gate features, odd rows the matching up features: the two
        // lanes of a pair swap halves of their 16 columns, the even lane finishes columns
        // 0..7 and the odd lane columns 8..15 of silu(gate) * up
        const bool odd = lane & 1;
        float other[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) other[jj] = __shfl_xor_sync(0xffffffffu, odd ? v[jj] : v[8 + jj], 1);
        const int f = (n0 >> 1) + (row >> 1);          // output feature
        if (f < p.N_out && waited) {
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                const float gte = odd ? other[jj] : v[jj], up = odd ? v[8 + jj] : other[jj];
                const int c = c0 + (odd ? 8 : 0) + jj;
                if (mine(c))
                    gb_store(p.out, p.out_dtype, size_t(t0 + c) * p.ldo + f, gte / (1.f + expf(-gte)) * up);
            }
        }
    }
}

// After tc_finish_chunk over the columns [c_begin, c_end) with a residual epilogue: the tile's sums of
// squares per token, for the norm that comes next.
template <int BN>
__device__ __forceinline__ void tc_write_ssq(const TcParams& p, int n0, int t0, int row, int c_begin, int c_end,
                                             float (*ssq_s)[BN]) {
    asm volatile("bar.sync 1, 128;" ::: "memory");
    for (int c = c_begin + row; c < c_end; c += 128)
        p.ssq_out[size_t(n0 / BM) * p.T + t0 + c] = ssq_s[0][c] + ssq_s[1][c] + ssq_s[2][c] + ssq_s[3][c];
    asm volatile("bar.sync 1, 128;" ::: "memory");     // ssq_s is written again by the next unit
}

}  // namespace

// Two CTAs on two SMs per 256 x 256 tile (gemm_tc_pair.cu); taken for steps of many tokens.
// mo: map of the bf16 output for stores from shared memory (boxes of 16 tokens x 128 features, or x 64 after
// SwiGLU), or null: results are then stored from registers.
int gemm_tc_pair_launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap* mo, const void* params,
                        cudaStream_t stream);
