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
//                     four neighbouring lanes share a column (each keeps a quarter of its rows in registers) and
//                     add their parts of o with two shuffles.  Tokens are staged in shared memory sixteen at a time,
//                     the next sixteen requested while these are worked through.
// tb_gated_rmsnorm    y = o / sqrt(mean(o^2) + eps) * w * sigmoid(g) over the concatenated heads, one block a token.
#include "common.cuh"

struct LightningArgs {
    const void* proj; int stride;           // [T][stride]: q (H*dk) | k (H*dk) | v (H*dv) | g (H*dv), compute dtype
    float* out; int out_stride;             // [T][out_stride] float32: head h at h * dv
    float* state;                           // [slots][H][dk][dv] float32
    const float* decay;                     // [H]
    const int* q_start; const int* slot_of_seq;
    int B; int H; int dk; int dv;
    int max_new;                            // most tokens a sequence brings in this step (1: a step of single tokens)
};

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// CH tokens of a sequence are staged in shared memory at a time (q and k of the head with the activation applied, and the
// block's 32 value columns), requested into registers while the chunk before is worked through, so that the latency of
// the loads is paid once a chunk and not once a token.  Within a chunk the tokens are taken one after the other from
// shared memory: a thread keeps rows [s * R, (s + 1) * R) of its column of the state in registers (s = lane & 3), reads
// the matching q and k as 16-byte loads (rows of the four s are 16 bytes apart in the banks), and the four partial sums
// of o meet by two shuffles.
template <typename T, int R, int CH>
__global__ void __launch_bounds__(128) lightning_scan_kernel(LightningArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr int DKP = 4 * (R + 4);                    // a q or k row in shared memory: four runs of R, each padded by 4
    constexpr int ROW = 2 * DKP + 32;                   // q | k | 32 values
    constexpr int PER = (CH * ROW + 127) / 128;         // staged elements a thread
    const int b = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, s = tid & 3, col = tid >> 2, j = blockIdx.z * 32 + col;
    const int dk = a.dk, dv = a.dv;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    const bool live = j < dv;
    float* S_g = a.state + (((size_t)a.slot_of_seq[b] * a.H + h) * dk) * dv + j;
    float S[R];
#pragma unroll
    for (int ii = 0; ii < R; ++ii) {
        const int i = s * R + ii;
        S[ii] = (live && i < dk) ? S_g[(size_t)i * dv] : 0.f;
    }
    const float decay = a.decay[h];
    const T* base = (const T*)a.proj;
    const int kq = h * dk, kk = a.H * dk + h * dk, kvv = 2 * a.H * dk + h * dv + blockIdx.z * 32;
    float stage[PER];
    // element e of a chunk's staging area: token e / ROW, and within the row q (padded), k (padded) or a value
    auto request = [&](int first) {
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int e = tid + 128 * u, tok = e / ROW, x = e % ROW;
            float v = 0.f;
            if (e < CH * ROW && first + tok < t1) {
                const T* row = base + (size_t)(first + tok) * a.stride;
                if (x < 2 * DKP) {
                    const int y = x < DKP ? x : x - DKP, run = y / (R + 4), within = y % (R + 4), i = run * R + within;
                    if (within < R && i < dk) v = ldf(row + (x < DKP ? kq : kk) + i);
                } else if (blockIdx.z * 32 + (x - 2 * DKP) < dv) {
                    v = ldf(row + kvv + (x - 2 * DKP));
                }
            }
            stage[u] = v;
        }
    };
    if (t0 < t1) request(t0);
    for (int c0 = t0; c0 < t1; c0 += CH) {
        __syncthreads();                                // the chunk before has been read from shared memory
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int e = tid + 128 * u;
            if (e < CH * ROW) sm[e] = silu_f(stage[u]);   // silu(0) = 0: the padding stays zero
        }
        __syncthreads();
        if (c0 + CH < t1) request(c0 + CH);
        const int n = min(CH, t1 - c0);
        for (int tt = 0; tt < n; ++tt) {
            const float* qs = sm + tt * ROW + s * (R + 4);
            const float* ks = qs + DKP;
            const float vj = sm[tt * ROW + 2 * DKP + col];
            float acc = 0.f;
#pragma unroll
            for (int ii = 0; ii < R; ii += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(ks + ii), q4 = *reinterpret_cast<const float4*>(qs + ii);
                S[ii] = fmaf(decay, S[ii], k4.x * vj);         acc = fmaf(S[ii], q4.x, acc);
                S[ii + 1] = fmaf(decay, S[ii + 1], k4.y * vj); acc = fmaf(S[ii + 1], q4.y, acc);
                S[ii + 2] = fmaf(decay, S[ii + 2], k4.z * vj); acc = fmaf(S[ii + 2], q4.z, acc);
                S[ii + 3] = fmaf(decay, S[ii + 3], k4.w * vj); acc = fmaf(S[ii + 3], q4.w, acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (s == 0 && live) a.out[(size_t)(c0 + tt) * a.out_stride + h * dv + j] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int ii = 0; ii < R; ++ii) {
            const int i = s * R + ii;
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

template <typename T, int R, int CH>
int launch_one(const LightningArgs& a, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = (size_t)CH * (2 * 4 * (R + 4) + 32) * sizeof(float);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(lightning_scan_kernel<T, R, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        TB_REQUIRE(e == cudaSuccess, "lightning_scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    tb_launch(lightning_scan_kernel<T, R, CH>, grid, 128, smem, stream, a);
    return 0;
}

// Rows of the state a thread keeps (a quarter of dk, rounded up to 8, 16, 32 or 64) and tokens staged at a time: sixteen for
// prompts, one for steps of single tokens (nothing to amortise, and less to request).
template <typename T>
int launch_scan(const LightningArgs& a, bool single, cudaStream_t stream) {
    dim3 grid(a.B, a.H, (a.dv + 31) / 32);
    const int rows = (a.dk + 3) / 4;
    if (single) {
        if (rows <= 8) return launch_one<T, 8, 1>(a, grid, stream);
        if (rows <= 16) return launch_one<T, 16, 1>(a, grid, stream);
        if (rows <= 32) return launch_one<T, 32, 1>(a, grid, stream);
        return launch_one<T, 64, 1>(a, grid, stream);
    }
    if (rows <= 8) return launch_one<T, 8, 16>(a, grid, stream);
    if (rows <= 16) return launch_one<T, 16, 16>(a, grid, stream);
    if (rows <= 32) return launch_one<T, 32, 16>(a, grid, stream);
    return launch_one<T, 64, 8>(a, grid, stream);
}

}  // namespace

extern "C" int tb_lightning_scan(const LightningArgs* args, int dtype, cudaStream_t stream) {
    LightningArgs a = *args;
    TB_REQUIRE(a.B > 0 && a.H > 0 && a.dk > 0 && a.dv > 0, "lightning_scan: sizes must be positive");
    TB_REQUIRE(a.dk <= 256, "lightning_scan: %d key dimensions a head (at most 256)", a.dk);
    TB_REQUIRE(a.H <= 65535 && (a.dv + 31) / 32 <= 65535, "lightning_scan: too many heads or value columns");
    TB_REQUIRE(a.proj && a.out && a.state && a.decay && a.q_start && a.slot_of_seq, "lightning_scan: missing buffers");
    TB_REQUIRE(a.stride >= 2 * a.H * a.dk + a.H * a.dv, "lightning_scan: the projection row is too short");
    TB_REQUIRE(dtype == TB_F32 || dtype == TB_BF16, "lightning_scan: unknown dtype %d", dtype);
    const bool single = a.max_new <= 1;
    if (dtype == TB_F32 ? launch_scan<float>(a, single, stream) : launch_scan<__nv_bfloat16>(a, single, stream)) return 1;
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
