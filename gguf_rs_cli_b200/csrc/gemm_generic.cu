// Plain matrix product on the CUDA cores: out[t,n] = sum_k X[t,k] * W[n,k] (+ bias[n]),
// W row-major [out, in] as the reference stores it (src/tensor/dequant.rs:258-259,
// 315-317).  Every product and sum is a 32-bit FMA; each output element is summed by
// one thread in ascending k, so a row's result does not depend on which other rows
// are in the batch.  It is the whole matrix path of the 32-bit mode, the twin that
// the tensor-core kernel is tested against, and the path for sizes the tensor-core
// kernel refuses.
#include "common.cuh"

constexpr int GG_BM = 64, GG_BN = 64, GG_BK = 16;

template <typename TX, typename TW>
__global__ void __launch_bounds__(256) gemm_generic_kernel(const TX* __restrict__ X, long long ldx,
                                                           const TW* __restrict__ W, long long ldw,
                                                           const void* __restrict__ bias, int bias_dtype,
                                                           void* __restrict__ out, int out_dtype, long long ldo, int T,
                                                           int N, int K) {
    __shared__ float Xs[GG_BK][GG_BM + 4];
    __shared__ float Ws[GG_BK][GG_BN + 4];
    int tid = threadIdx.x;
    int tx = tid & 15, ty = tid >> 4;
    int t0 = blockIdx.y * GG_BM, n0 = blockIdx.x * GG_BN;
    int lrow = tid >> 2, lk = (tid & 3) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GG_BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int k = k0 + lk + j;
            int t = t0 + lrow, n = n0 + lrow;
            Xs[lk + j][lrow] = (t < T && k < K) ? gb_to_float(X[size_t(t) * ldx + k]) : 0.f;
            Ws[lk + j][lrow] = (n < N && k < K) ? gb_to_float(W[size_t(n) * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = Xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += gb_load(bias, bias_dtype, n);
            gb_store(out, out_dtype, size_t(t) * ldo + n, v);
        }
    }
}

GB_API int gb_gemm_generic(const void* X, int x_dtype, long long ldx, const void* W, int w_dtype, long long ldw,
                           const void* bias, int bias_dtype, void* out, int out_dtype, long long ldo, int T, int N,
                           int K, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(x_dtype) && gb_is_dtype(w_dtype) && gb_is_dtype(out_dtype), "gb_gemm_generic: bad dtype");
    GB_REQUIRE(!bias || gb_is_dtype(bias_dtype), "gb_gemm_generic: bad bias dtype");
    GB_REQUIRE(T >= 0 && N > 0 && K > 0 && ldx >= K && ldw >= K && ldo >= N,
               "gb_gemm_generic: bad sizes T=%d N=%d K=%d ldx=%lld ldw=%lld ldo=%lld", T, N, K, ldx, ldw, ldo);
    if (T == 0) return 0;
    dim3 grid((N + GG_BN - 1) / GG_BN, (T + GG_BM - 1) / GG_BM);
    GB_REQUIRE(grid.y <= 65535, "gb_gemm_generic: T=%d is too many rows for one launch", T);
#define GG_LAUNCH(TX, TW)                                                                                           \
    gemm_generic_kernel<TX, TW><<<grid, 256, 0, stream>>>((const TX*)X, ldx, (const TW*)W, ldw, bias, bias_dtype, out, \
                                                          out_dtype, ldo, T, N, K)
    if (x_dtype == GB_F32 && w_dtype == GB_F32) GG_LAUNCH(float, float);
    else if (x_dtype == GB_BF16 && w_dtype == GB_BF16) GG_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == GB_BF16 && w_dtype == GB_F32) GG_LAUNCH(__nv_bfloat16, float);
    else GG_LAUNCH(float, __nv_bfloat16);
#undef GG_LAUNCH
    GB_LAUNCH_OK("gb_gemm_generic");
    return 0;
}
