// Linear attention with a per-head decay ("lightning" mixer): the recurrence and the gated norm after it.
//
//   S_t = decay_h S_{t-1} + k_t v_t^T        S: [dk][dv] float32 per (sequence, head), kept in the cache's state group
//   o_t = S_t^T q_t
// with q = silu(.), k = silu(.), v = silu(.) of the projection's columns (the projection may be in the compute
// dtype; the activation, the state and the sums are float32).  A sequence's tokens are taken in order, so a prompt
// run whole, in pieces or token by token leaves the same state up to the order of float32 sums (which is the same
// here: one token after the other in every case).
//
// tb_lightning_scan   grid (sequences, heads, ceil(dv / 32)): a block owns 32 value columns of one head's state;
//                     four neighbouring lanes share a column (each keeps every fourth row of it in registers) and
//                     add their parts of o with two shuffles.  The next token's q, k and v are requested before
//                     the current token's arithmetic.
// tb_gated_rmsnorm    y = o / sqrt(mean(o^2) + eps) * w * sigmoid(g) over the concatenated heads, one block a token.
#include "common.cuh"

struct LightningArgs {
    const void* proj; int stride;           // [T][stride]: q (H*dk) | k (H*dk) | v (H*dv) | g (H*dv), compute dtype
    float* out; int out_stride;             // [T][out_stride] float32: head h at h * dv
    float* state;                           // [slots][H][dk][dv] float32
    const float* decay;                     // [H]
    const int* q_start; const int* slot_of_seq;
    int B; int H; int dk; int dv;
};

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

template <typename T, int R>
__global__ void __launch_bounds__(128) lightning_scan_kernel(LightningArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];           // q [dk], k [dk]
    const int b = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, s = tid & 3, j = blockIdx.z * 32 + (tid >> 2);
    const int dk = a.dk, dv = a.dv;
    float* qs = sm;
    float* ks = sm + dk;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    const bool live = j < dv;
    float* S_g = a.state + (((size_t)a.slot_of_seq[b] * a.H + h) * dk) * dv + j;
    float S[R];
#pragma unroll
    for (int ii = 0; ii < R; ++ii) {
        const int i = s + 4 * ii;
        S[ii] = (live && i < dk) ? S_g[(size_t)i * dv] : 0.f;
    }
    const float decay = a.decay[h];
    const T* base = (const T*)a.proj;
    const int kq = h * dk, kk = a.H * dk + h * dk, kvv = 2 * a.H * dk + h * dv;
    // two of q and two of k a thread cover dk <= 256
    float nq[2], nk[2], nv = 0.f;
    auto request = [&](int t) {
        const T* row = base + (size_t)t * a.stride;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int i = tid + 128 * u;
            nq[u] = i < dk ? ldf(row + kq + i) : 0.f;
            nk[u] = i < dk ? ldf(row + kk + i) : 0.f;
        }
        nv = live ? ldf(row + kvv + j) : 0.f;
    };
    if (t0 < t1) request(t0);
    for (int t = t0; t < t1; ++t) {
        __syncthreads();                    // the token before has been read from shared memory
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int i = tid + 128 * u;
            if (i < dk) { qs[i] = silu_f(nq[u]); ks[i] = silu_f(nk[u]); }
        }
        const float vj = silu_f(nv);
        __syncthreads();
        if (t + 1 < t1) request(t + 1);
        float acc = 0.f;
#pragma unroll
        for (int ii = 0; ii < R; ++ii) {
            const int i = s + 4 * ii;
            if (i < dk) {
                S[ii] = fmaf(decay, S[ii], ks[i] * vj);
                acc = fmaf(S[ii], qs[i], acc);
            }
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (s == 0 && live) a.out[(size_t)t * a.out_stride + h * dv + j] = acc;
    }
    if (live) {
#pragma unroll
        for (int ii = 0; ii < R; ++ii) {
            const int i = s + 4 * ii;
            if (i < dk) S_g[(size_t)i * dv] = S[ii];
        }
    }
}

template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ w, const T* __restrict__ gate,
                                     int ldg, T* __restrict__ y, int ldy, int N, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t t = blockIdx.x;
    const float* row = o + t * ldo;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) ss += row[i] * row[i];
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float g = ldf(gate + t * ldg + i);
        stf(y + t * ldy + i, row[i] * scale * w[i] * (1.0f / (1.0f + expf(-g))));
    }
}

template <typename T>
int launch_scan(const LightningArgs& a, cudaStream_t stream) {
    dim3 grid(a.B, a.H, (a.dv + 31) / 32);
    const size_t smem = 2 * (size_t)a.dk * sizeof(float);
    const int rows = (a.dk + 3) / 4;
    if (rows <= 8) tb_launch(lightning_scan_kernel<T, 8>, grid, 128, smem, stream, a);
    else if (rows <= 16) tb_launch(lightning_scan_kernel<T, 16>, grid, 128, smem, stream, a);
    else if (rows <= 32) tb_launch(lightning_scan_kernel<T, 32>, grid, 128, smem, stream, a);
    else tb_launch(lightning_scan_kernel<T, 64>, grid, 128, smem, stream, a);
    return 0;
}

}  // namespace

extern "C" int tb_lightning_scan(const LightningArgs* args, int dtype, cudaStream_t stream) {
    LightningArgs a = *args;
    TB_REQUIRE(a.B > 0 && a.H > 0 && a.dk > 0 && a.dv > 0, "lightning_scan: sizes must be positive");
    TB_REQUIRE(a.dk <= 256, "lightning_scan: %d key dimensions a head (at most 256)", a.dk);
    TB_REQUIRE(a.H <= 65535 && (a.dv + 31) / 32 <= 65535, "lightning_scan: too many heads or value columns");
    TB_REQUIRE(a.proj && a.out && a.state && a.decay && a.q_start && a.slot_of_seq, "lightning_scan: missing buffers");
    TB_REQUIRE(a.stride >= 2 * a.H * a.dk + a.H * a.dv, "lightning_scan: the projection row is too short");
    if (dtype == TB_F32) launch_scan<float>(a, stream);
    else if (dtype == TB_BF16) launch_scan<__nv_bfloat16>(a, stream);
    else TB_REQUIRE(false, "lightning_scan: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("lightning_scan");
    return 0;
}

extern "C" int tb_gated_rmsnorm(const float* o, int ldo, const float* w, const void* gate, int ldg, void* y, int ldy,
                                int dtype, int n_rows, int N, float eps, cudaStream_t stream) {
    TB_REQUIRE(n_rows > 0 && N > 0 && o && w && gate && y, "gated_rmsnorm: sizes must be positive (rows=%d N=%d)", n_rows, N);
    const int threads = N >= 2048 ? 256 : (N >= 512 ? 128 : 64);
    if (dtype == TB_F32) tb_launch(gated_rmsnorm_kernel<float>, n_rows, threads, 0, stream, o, ldo, w, (const float*)gate, ldg, (float*)y, ldy, N, eps);
    else if (dtype == TB_BF16) tb_launch(gated_rmsnorm_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, o, ldo, w, (const __nv_bfloat16*)gate, ldg, (__nv_bfloat16*)y, ldy, N, eps);
    else TB_REQUIRE(false, "gated_rmsnorm: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("gated_rmsnorm");
    return 0;
}
