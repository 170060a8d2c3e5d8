// Plain matrix product on the CUDA cores: out = X[M,K] . W[N,K]^T with float32 accumulation.
//
// This is the true 32-bit path (T = float: FFMA only, no tensor-core or reduced-precision mode)
// and the plain twin of the tensor-core kernel for bfloat16 operands; it takes every M, N, K.
// berniehans/titan's counterpart is its warp-per-column kernels
// (engine/engine-cuda/kernels/gemm_quant.cu:2331-2363 gemm_f32_kernel, :3365-3499 batched), which
// fuse the residual into the epilogue (:3489-3493) and SwiGLU into gate/up (:2589).
//
// Epilogues:
//   TB_EPI_STORE   out[m][n] = acc                      (compute dtype)
//   TB_EPI_F32     out[m][n] = acc                      (float32: logits)
//   TB_EPI_ADD     out[m][n] += acc                     (float32 residual stream, in place)
//   TB_EPI_SWIGLU  out[m][j] = gate(acc[2j], acc[2j+1]) (rows of W interleaved gate, up; N even); the gate is
//                  silu(g) * u unless the launch names another (activation.h)
#include "common.cuh"
#include "gemm.h"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ X, const T* __restrict__ W, void* __restrict__ out_,
                 int M, int N, int K, int ldx, int ldo, long long sx, long long sw, long long so, int act, float limit) {
    pdl_launch_dependents();
    pdl_wait();
    // blockIdx.z: one of a batch of products of equal shape (the heads of a mixer, say), each at its own offset
    X += (size_t)blockIdx.z * sx;
    W += (size_t)blockIdx.z * sw;
    void* out = (EPI == TB_EPI_STORE || EPI == TB_EPI_SWIGLU) ? (void*)((T*)out_ + (size_t)blockIdx.z * so)
                                                              : (void*)((float*)out_ + (size_t)blockIdx.z * so);
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;     // thread tile: rows ty*4.., cols tx*4..
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k of each operand: 1024 elements, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx / BK, kk = idx % BK;
            const int k = k0 + kk;
            xs[kk][r] = (m0 + r < M && k < K) ? ldf(X + (size_t)(m0 + r) * ldx + k) : 0.f;
            ws[kk][r] = (n0 + r < N && k < K) ? ldf(W + (size_t)(n0 + r) * K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
        if (EPI == TB_EPI_SWIGLU) {
#pragma unroll
            for (int j = 0; j < TN; j += 2) {
                const int n = n0 + tx * TN + j;
                if (n + 1 < N) {
                    const float g = acc[i][j], u = acc[i][j + 1];
                    stf((T*)out + (size_t)m * ldo + n / 2, tb_gated(act, limit, g, u));
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int n = n0 + tx * TN + j;
                if (n >= N) continue;
                if (EPI == TB_EPI_STORE) stf((T*)out + (size_t)m * ldo + n, acc[i][j]);
                if (EPI == TB_EPI_F32) ((float*)out)[(size_t)m * ldo + n] = acc[i][j];
                if (EPI == TB_EPI_ADD) ((float*)out)[(size_t)m * ldo + n] += acc[i][j];
            }
        }
    }
}

template <typename T>
int launch(const void* X, const void* W, void* out, int M, int N, int K, int ldx, int ldo, int epi,
           int batch, long long sx, long long sw, long long so, int act, float limit, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
    const T* x = (const T*)X;
    const T* w = (const T*)W;
    switch (epi) {
        case TB_EPI_STORE: tb_launch(gemm_simt_kernel<T, TB_EPI_STORE>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo, sx, sw, so, act, limit); break;
        case TB_EPI_F32: tb_launch(gemm_simt_kernel<T, TB_EPI_F32>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo, sx, sw, so, act, limit); break;
        case TB_EPI_ADD: tb_launch(gemm_simt_kernel<T, TB_EPI_ADD>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo, sx, sw, so, act, limit); break;
        case TB_EPI_SWIGLU: tb_launch(gemm_simt_kernel<T, TB_EPI_SWIGLU>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo, sx, sw, so, act, limit); break;
        default: tb_set_error("gemm: unknown epilogue %d", epi); return 1;
    }
    return 0;
}

// A few rows (decode steps): a warp per output element of one row and one product of the batch, lanes along K with
// 16-byte loads where the rows allow; the weights are read once per row of X through L2.  Epilogues STORE, F32 and ADD.
template <typename T, int EPI>
__global__ void __launch_bounds__(256)
gemm_rows_kernel(const T* __restrict__ X, const T* __restrict__ W, void* __restrict__ out_, int M, int N, int K, int ldx, int ldo,
                 long long sx, long long sw, long long so) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * 8 + warp, m = blockIdx.y, z = blockIdx.z;
    if (n >= N) return;
    const T* x = X + (size_t)z * sx + (size_t)m * ldx;
    const T* w = W + (size_t)z * sw + (size_t)n * K;
    constexpr int PER = 16 / sizeof(T);
    float acc = 0.f;
    if (K % PER == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0)) {
        for (int k = lane * PER; k < K; k += 32 * PER) {
            if (sizeof(T) == 4) {
                const float4 a = *reinterpret_cast<const float4*>(x + k), b = *reinterpret_cast<const float4*>(w + k);
                acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
            } else {
                const uint4 a = *reinterpret_cast<const uint4*>(x + k), b = *reinterpret_cast<const uint4*>(w + k);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(bw[i] << 16), acc);
                    acc = fmaf(__uint_as_float(aw[i] & 0xffff0000u), __uint_as_float(bw[i] & 0xffff0000u), acc);
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(ldf(x + k), ldf(w + k), acc);
    }
    acc = warp_sum(acc);
    if (lane != 0) return;
    const size_t at = (size_t)z * so + (size_t)m * ldo + n;
    if (EPI == TB_EPI_STORE) stf((T*)out_ + at, acc);
    if (EPI == TB_EPI_F32) ((float*)out_)[at] = acc;
    if (EPI == TB_EPI_ADD) ((float*)out_)[at] += acc;
}

template <typename T>
static int launch_rows(const void* X, const void* W, void* out, int M, int N, int K, int ldx, int ldo, int epi, int batch,
                       long long sx, long long sw, long long so, cudaStream_t stream) {
    dim3 grid((N + 7) / 8, M, batch);
    const T* x = (const T*)X;
    const T* w = (const T*)W;
    if (epi == TB_EPI_STORE) tb_launch(gemm_rows_kernel<T, TB_EPI_STORE>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo, sx, sw, so);
    else if (epi == TB_EPI_F32) tb_launch(gemm_rows_kernel<T, TB_EPI_F32>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo, sx, sw, so);
    else if (epi == TB_EPI_ADD) tb_launch(gemm_rows_kernel<T, TB_EPI_ADD>, grid, 256, 0, stream, x, w, out, M, N, K, ldx, ldo, sx, sw, so);
    else { tb_set_error("gemm_rows: epilogue %d is not one of store, float32, add", epi); return 1; }
    return 0;
}

}  // namespace

// ldx: row stride of X in elements; ldo: row stride of out in elements.  ``batch`` products of the same shape in one
// launch: product z reads X + z * sx and W + z * sw and writes out + z * so (offsets in elements).
// act, limit: the gate of the SWIGLU epilogue (activation.h).
extern "C" int tb_gemm_simt_gated(const void* X, const void* W, void* out, int dtype, int M, int N, int K, int ldx,
                                  int ldo, int epi, int batch, long long sx, long long sw, long long so, int act, float limit,
                                  cudaStream_t stream) {
    TB_REQUIRE(act >= 0 && act < TB_ACT_KINDS, "gemm: unknown gate %d", act);
    TB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: sizes must be positive (M=%d N=%d K=%d)", M, N, K);
    TB_REQUIRE(batch > 0 && batch <= 65535, "gemm: a batch of %d products", batch);
    TB_REQUIRE(ldx >= K, "gemm: row stride %d of X is shorter than K=%d", ldx, K);
    TB_REQUIRE(epi != TB_EPI_SWIGLU || N % 2 == 0, "gemm: the SwiGLU epilogue needs an even N, found %d", N);
    TB_REQUIRE((M + BM - 1) / BM <= 65535, "gemm: M=%d is too large for one launch", M);
    if (epi == TB_EPI_STORE && M <= 16 && batch > 1 && (N + 7) / 8 <= 65535) {      // a decode step's rows: a warp per output
        int r;
        if (dtype == TB_F32) r = launch_rows<float>(X, W, out, M, N, K, ldx, ldo, epi, batch, sx, sw, so, stream);
        else if (dtype == TB_BF16) r = launch_rows<__nv_bfloat16>(X, W, out, M, N, K, ldx, ldo, epi, batch, sx, sw, so, stream);
        else { tb_set_error("gemm: unknown dtype %d", dtype); return 1; }
        if (r) return r;
        TB_CHECK_LAUNCH("gemm_rows");
        return 0;
    }
    int rc;
    if (dtype == TB_F32) rc = launch<float>(X, W, out, M, N, K, ldx, ldo, epi, batch, sx, sw, so, act, limit, stream);
    else if (dtype == TB_BF16) rc = launch<__nv_bfloat16>(X, W, out, M, N, K, ldx, ldo, epi, batch, sx, sw, so, act, limit, stream);
    else { tb_set_error("gemm: unknown dtype %d", dtype); return 1; }
    if (rc) return rc;
    TB_CHECK_LAUNCH("gemm_simt");
    return 0;
}

extern "C" int tb_gemm_simt_batched(const void* X, const void* W, void* out, int dtype, int M, int N, int K, int ldx,
                                    int ldo, int epi, int batch, long long sx, long long sw, long long so, cudaStream_t stream) {
    return tb_gemm_simt_gated(X, W, out, dtype, M, N, K, ldx, ldo, epi, batch, sx, sw, so, TB_ACT_SILU, 0.f, stream);
}

extern "C" int tb_gemm_simt(const void* X, const void* W, void* out, int dtype, int M, int N, int K, int ldx,
                            int ldo, int epi, cudaStream_t stream) {
    return tb_gemm_simt_batched(X, W, out, dtype, M, N, K, ldx, ldo, epi, 1, 0, 0, 0, stream);
}

// out (epilogue store, float32 or add) = X[M,K] . W[N,K]^T for a few rows and a small matrix, a warp per output element:
// the products of a decode step whose matrices are too small to pay for a tensor-core launch (a router, a narrow gate).
extern "C" int tb_gemm_rows(const void* X, const void* W, void* out, int dtype, int M, int N, int K, int ldx, int ldo, int epi,
                            cudaStream_t stream) {
    TB_REQUIRE(M > 0 && N > 0 && K > 0 && M <= 65535 && (N + 7) / 8 <= 2147483647, "gemm_rows: sizes (M=%d N=%d K=%d)", M, N, K);
    TB_REQUIRE(ldx >= K, "gemm_rows: row stride %d of X is shorter than K=%d", ldx, K);
    int r;
    if (dtype == TB_F32) r = launch_rows<float>(X, W, out, M, N, K, ldx, ldo, epi, 1, 0, 0, 0, stream);
    else if (dtype == TB_BF16) r = launch_rows<__nv_bfloat16>(X, W, out, M, N, K, ldx, ldo, epi, 1, 0, 0, 0, stream);
    else { tb_set_error("gemm_rows: unknown dtype %d", dtype); return 1; }
    if (r) return r;
    TB_CHECK_LAUNCH("gemm_rows");
    return 0;
}
