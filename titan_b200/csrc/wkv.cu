// The "wkv" mixer: a linear recurrence whose decay is made from the token itself, with a bonus for the current token.
//
//   mix_s[t] = h[t] + (h[t-1] - h[t]) * mu_s        s in r, k, v, g, w; h[-1] is the last row of the step before (zero at the start)
//   w[t]     = exp(-exp(W2 tanh(W1 mix_w[t]) + w0))  per head and key channel, float32
//   o[t]     = (S + diag(u) k[t] v[t]^T)^T r[t]      per head; S: [dk][dk] float32 (key x value)
//   S        = diag(w[t]) S + k[t] v[t]^T
//   y[t]     = o[t] / rms(o[t]) per head, * weight * silu(g[t])
//
// A sequence's state (every head's S, then the last input row) lies in one float32 row of the cache's state group.  The
// projections r, k, v, g and W1 mix_w are matrix products of the compute dtype; everything that enters the recurrence
// after them is float32 here: the decay and its two exponentials, the bonus, the state, the sums and the unit norm.
//
//   tb_wkv_shift   the five mixes of every token, side by side in one row (a block a token)
//   tb_wkv_decay   w of every token and channel from the low-rank product's first half (tanh, the second product, w0, exp(-exp))
//   tb_wkv_scan    the recurrence; grid (sequences, heads, ceil(dk / 32 or 16)): a block owns 32 (or 16) value columns of one
//                  head's state, four (or eight) neighbouring lanes share a column (a share of its rows each, in registers)
//                  and add their parts of o by shuffles; tokens are staged in shared memory a chunk at a time, the next chunk's loads in
//                  flight while this one is worked through.  Tokens are taken in order whatever the step brings, so a
//                  prompt run whole, in pieces or token by token leaves the same state.  The block of head 0 also
//                  leaves the sequence's last input row in the state.
//   tb_wkv_out     unit RMS of every head's o, the weight and the gate (a warp a token and head)
#include "common.cuh"

struct WkvArgs {
    const void* h; int h_stride;            // [T][h_stride] the mixer's input rows (compute dtype), W wide
    void* mixes; int mix_stride;            // [T][mix_stride]: mix_r | mix_k | mix_v | mix_g | mix_w, each W wide (compute dtype)
    const float* mu;                        // [5][W]
    const void* proj; int proj_stride;      // [T][proj_stride]: r | k | v | g, each H * dk wide (compute dtype)
    const void* lora; int lora_stride;      // [T][lora_stride]: W1 mix_w, rank wide (compute dtype)
    const void* w2;                         // [H * dk][rank] (compute dtype)
    const float* w0;                        // [H * dk]
    float* decay;                           // [T][H * dk] float32
    const float* u;                         // [H][dk]
    float* out; int out_stride;             // [T][out_stride] float32: head h at h * dk
    float* state; long long state_stride;   // [slots][state_stride]: S [H][dk][dk], then the last input row [W]
    const float* norm_w;                    // [H * dk]
    void* y; int y_stride;                  // [T][y_stride] (compute dtype)
    float eps;
    const int* q_start; const int* slot_of_seq; const int* seq_of;
    int T; int B; int H; int dk; int W; int rank; int max_new;
};

namespace {

// Eight consecutive elements of a row as floats, from one (bfloat16) or two (float32) 16-byte accesses.
template <typename T> __device__ __forceinline__ void load8(const T* p, float* o);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* o) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* v);
template <> __device__ __forceinline__ void store8<float>(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 q = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&q);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// VEC: rows, strides and pointers allow 16-byte accesses of eight elements (the launcher checks); else element by element.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) wkv_shift_kernel(WkvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, seq = a.seq_of[t];
    const bool first = t == a.q_start[seq];
    const T* cur = (const T*)a.h + (size_t)t * a.h_stride;
    const T* before = cur - a.h_stride;
    const float* last = a.state + (size_t)a.slot_of_seq[seq] * a.state_stride + (size_t)a.H * a.dk * a.dk;
    T* out = (T*)a.mixes + (size_t)t * a.mix_stride;
    constexpr int E = VEC ? 8 : 1;
    const int units = a.W / E;                          // gridDim.y blocks share a row
    const int per = (units + gridDim.y - 1) / gridDim.y, u0 = blockIdx.y * per, u1 = min(units, u0 + per);
    for (int u = u0 + threadIdx.x; u < u1; u += blockDim.x) {
        const int i = u * E;
        float x[E], p[E];
        if (VEC) {
            load8<T>(cur + i, x);
            if (first) {                                 // (the state's row is float32 and need not be 16-byte aligned)
#pragma unroll
                for (int k = 0; k < E; ++k) p[k] = last[i + k];
            } else load8<T>(before + i, p);
        } else {
            x[0] = ldf(cur + i);
            p[0] = first ? last[i] : ldf(before + i);
        }
#pragma unroll
        for (int s = 0; s < 5; ++s) {
            float m[E], o[E];
            if (VEC) load8<float>(a.mu + (size_t)s * a.W + i, m);
            else m[0] = a.mu[(size_t)s * a.W + i];
#pragma unroll
            for (int k = 0; k < E; ++k) o[k] = x[k] + (p[k] - x[k]) * m[k];
            if (VEC) store8<T>(out + (size_t)s * a.W + i, o);
            else stf(out + (size_t)s * a.W + i, o[0]);
        }
    }
}

// A block takes DEC_TOK tokens and 128 channels: the channels' rows of W2 and the tokens' tanh rows go through shared
// memory in pieces of DEC_J columns of the rank (W2 rows padded by one against bank conflicts), so W2 is read once per
// DEC_TOK tokens and every read of it is along its rows.
#define DEC_TOK 16
#define DEC_J 64
template <typename T>
__global__ void __launch_bounds__(128) wkv_decay_kernel(WkvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float w2s[128][DEC_J + 1];
    __shared__ float ths[DEC_TOK][DEC_J];
    const int N = a.H * a.dk, tid = threadIdx.x;
    const int t0 = blockIdx.x * DEC_TOK, n0 = blockIdx.y * 128, n = n0 + tid;
    const int n_tok = min(DEC_TOK, a.T - t0);
    float acc[DEC_TOK];
#pragma unroll
    for (int t = 0; t < DEC_TOK; ++t) acc[t] = 0.f;
    for (int j0 = 0; j0 < a.rank; j0 += DEC_J) {
        const int nj = min(DEC_J, a.rank - j0);
        __syncthreads();
        for (int e = tid; e < 128 * DEC_J; e += 128) {
            const int r = e / DEC_J, j = e % DEC_J;
            w2s[r][j] = (n0 + r < N && j < nj) ? ldf((const T*)a.w2 + (size_t)(n0 + r) * a.rank + j0 + j) : 0.f;
        }
        for (int e = tid; e < DEC_TOK * DEC_J; e += 128) {
            const int t = e / DEC_J, j = e % DEC_J;
            ths[t][j] = (t < n_tok && j < nj) ? tanhf(ldf((const T*)a.lora + (size_t)(t0 + t) * a.lora_stride + j0 + j)) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int j = 0; j < DEC_J; ++j) {
            const float wv = w2s[tid][j];
#pragma unroll
            for (int t = 0; t < DEC_TOK; ++t) acc[t] = fmaf(wv, ths[t][j], acc[t]);
        }
    }
    if (n >= N) return;
    const float w0 = a.w0[n];
#pragma unroll
    for (int t = 0; t < DEC_TOK; ++t)
        if (t < n_tok) a.decay[(size_t)(t0 + t) * N + n] = expf(-expf(acc[t] + w0));
}

// LPC lanes share a column of the state (R rows of it each: dk <= LPC * R), so a block of 128 threads owns COLS = 128 / LPC
// value columns.  Four lanes a column where the launch has blocks enough to fill the machine; eight (half the rows a thread,
// twice the blocks) where it has not: a token's chain of dependent sums is then half as long.
template <typename T, int R, int CH, int LPC>
__global__ void __launch_bounds__(128) wkv_scan_kernel(WkvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr int COLS = 128 / LPC;
    constexpr int DKP = LPC * (R + 4);                  // a row of dk numbers in shared memory: LPC runs of R, each padded by 4
    constexpr int ROW = 4 * DKP + COLS;                 // r | k | w | r * u | the block's values
    const int b = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, s = tid % LPC, col = tid / LPC, j = blockIdx.z * COLS + col;
    const int dk = a.dk, N = a.H * dk;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    const bool live = j < dk;
    float* slot_state = a.state + (size_t)a.slot_of_seq[b] * a.state_stride;
    float* S_g = slot_state + ((size_t)h * dk) * dk + j;
    float S[R];
#pragma unroll
    for (int ii = 0; ii < R; ++ii) {
        const int i = s * R + ii;
        S[ii] = (live && i < dk) ? S_g[(size_t)i * dk] : 0.f;
    }
    const T* proj = (const T*)a.proj;
    const float* bonus = a.u + (size_t)h * dk;
    // Staging.  A token's row of the chunk has 3 dk + COLS elements: r, k, w (dk each) and the block's values.  A thread
    // takes columns tid, tid + 128, ... of every token of the chunk; what a column is (which array, where it comes from,
    // where it goes in shared memory, its bonus) is worked out once, before the first chunk, so that the loop over chunks
    // divides nothing.  Loads are from valid addresses in every case (rows are clamped), so they carry no condition.
    constexpr int XI = (3 * LPC * R + COLS + 127) / 128;
    const int per_tok = 3 * dk + COLS;
    int src[XI], to[XI];            // column in the source row (r, k, v: of proj; w: of decay); offset in a token's shared row; to < 0: no such column
    bool from_decay[XI];
    float bonus_of[XI];             // r only: the bonus of its channel (its product goes 3 DKP further on); else 0 and unused
    bool is_r[XI];
#pragma unroll
    for (int xi = 0; xi < XI; ++xi) {
        const int x = tid + 128 * xi;
        src[xi] = 0; to[xi] = -1; from_decay[xi] = false; bonus_of[xi] = 0.f; is_r[xi] = false;
        if (x < 3 * dk) {
            const int arr = x / dk, i = x - arr * dk;
            to[xi] = arr * DKP + (i / R) * (R + 4) + (i % R);
            from_decay[xi] = arr == 2;
            src[xi] = arr == 2 ? h * dk + i : arr * N + h * dk + i;
            if (arr == 0) { is_r[xi] = true; bonus_of[xi] = bonus[i]; }
        } else if (x < per_tok) {
            const int c = x - 3 * dk;
            if (blockIdx.z * COLS + c < dk) { to[xi] = 4 * DKP + c; src[xi] = 2 * N + h * dk + blockIdx.z * COLS + c; }
        }
    }
    float stage[XI][CH];
    auto fetch = [&](int first) {
#pragma unroll
        for (int xi = 0; xi < XI; ++xi)
#pragma unroll
            for (int tok = 0; tok < CH; ++tok) {
                const size_t row = (size_t)min(first + tok, t1 - 1);
                stage[xi][tok] = from_decay[xi] ? a.decay[row * N + src[xi]] : ldf(proj + row * a.proj_stride + src[xi]);
            }
    };
    for (int e = tid; e < CH * ROW; e += 128) sm[e] = 0.f;       // the padding between runs and rows beyond dk are factors: zero
    if (t0 < t1) fetch(t0);
    for (int c0 = t0; c0 < t1; c0 += CH) {
        __syncthreads();                                // the chunk before has been read (or the zeros are in place)
#pragma unroll
        for (int xi = 0; xi < XI; ++xi) {
            if (to[xi] < 0) continue;
#pragma unroll
            for (int tok = 0; tok < CH; ++tok) {
                const float v = c0 + tok < t1 ? stage[xi][tok] : 0.f;
                sm[tok * ROW + to[xi]] = v;
                if (is_r[xi]) sm[tok * ROW + to[xi] + 3 * DKP] = v * bonus_of[xi];
            }
        }
        __syncthreads();
        if (c0 + CH < t1) fetch(c0 + CH);
        const int n = min(CH, t1 - c0);
        // (a block is one warp a scheduler: unrolled, the loads, sums and shuffles of neighbouring tokens overlap; only the
        // state's own update runs from token to token)
        constexpr int TOGETHER = R >= 32 ? 1 : 4;           // (eight were measured slower than four: 0.48 against 0.40 ms a layer)        // (wide heads hold too many rows a thread to hold several tokens as well)
#pragma unroll TOGETHER
        for (int tt = 0; tt < n; ++tt) {
            const float* rs = sm + tt * ROW + s * (R + 4);
            const float* ks = rs + DKP;
            const float* ws = ks + DKP;
            const float* us = ws + DKP;
            const float vj = sm[tt * ROW + 4 * DKP + col];
            float acc = 0.f, acc2 = 0.f, now = 0.f, now2 = 0.f;      // two chains each, so that a sum does not wait for the one before it
#pragma unroll
            for (int ii = 0; ii < R; ii += 4) {
                const float4 r4 = *reinterpret_cast<const float4*>(rs + ii), k4 = *reinterpret_cast<const float4*>(ks + ii);
                const float4 w4 = *reinterpret_cast<const float4*>(ws + ii), u4 = *reinterpret_cast<const float4*>(us + ii);
                acc = fmaf(S[ii], r4.x, acc);      now = fmaf(u4.x, k4.x, now);   S[ii] = fmaf(w4.x, S[ii], k4.x * vj);
                acc2 = fmaf(S[ii + 1], r4.y, acc2); now2 = fmaf(u4.y, k4.y, now2); S[ii + 1] = fmaf(w4.y, S[ii + 1], k4.y * vj);
                acc = fmaf(S[ii + 2], r4.z, acc);  now = fmaf(u4.z, k4.z, now);   S[ii + 2] = fmaf(w4.z, S[ii + 2], k4.z * vj);
                acc2 = fmaf(S[ii + 3], r4.w, acc2); now2 = fmaf(u4.w, k4.w, now2); S[ii + 3] = fmaf(w4.w, S[ii + 3], k4.w * vj);
            }
            acc = fmaf(now + now2, vj, acc + acc2);     // the current token's own pair, weighted by the bonus
#pragma unroll
            for (int o = 1; o < LPC; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (s == 0 && live) a.out[(size_t)(c0 + tt) * a.out_stride + h * dk + j] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int ii = 0; ii < R; ++ii) {
            const int i = s * R + ii;
            if (i < dk) S_g[(size_t)i * dk] = S[ii];
        }
    }
    if (h == 0 && blockIdx.z == 0 && t0 < t1) {         // the row that the next step's first token is mixed with
        float* last = slot_state + (size_t)a.H * dk * dk;
        const T* row = (const T*)a.h + (size_t)(t1 - 1) * a.h_stride;
        for (int i = tid; i < a.W; i += 128) last[i] = ldf(row + i);
    }
}

template <typename T>
__global__ void __launch_bounds__(128) wkv_out_kernel(WkvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x, h = blockIdx.y * 4 + warp;
    if (h >= a.H) return;
    const int dk = a.dk, N = a.H * dk;
    const float* o = a.out + (size_t)t * a.out_stride + h * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) ss += o[i] * o[i];
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)dk + a.eps);
    const T* g = (const T*)a.proj + (size_t)t * a.proj_stride + (size_t)3 * N + h * dk;
    T* y = (T*)a.y + (size_t)t * a.y_stride + h * dk;
    for (int i = lane; i < dk; i += 32) {
        const float gv = ldf(g + i);
        stf(y + i, o[i] * scale * a.norm_w[h * dk + i] * (gv / (1.0f + expf(-gv))));
    }
}

template <typename T, int R, int CH, int LPC>
cudaError_t launch_scan(const WkvArgs& a, cudaStream_t stream) {
    constexpr int COLS = 128 / LPC;
    constexpr size_t smem = (size_t)CH * (4 * LPC * (R + 4) + COLS) * sizeof(float);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        cudaFuncSetAttribute(wkv_scan_kernel<T, R, CH, LPC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        raised = true;
    }
    return tb_launch(wkv_scan_kernel<T, R, CH, LPC>, dim3(a.B, a.H, (a.dk + COLS - 1) / COLS), 128, smem, stream, a);
}

template <typename T>
int run(const WkvArgs& a, int stage, cudaStream_t stream) {
    if (stage == 0) {
        auto ok16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
        const bool vec = a.W % 8 == 0 && a.h_stride % 8 == 0 && a.mix_stride % 8 == 0 && ok16(a.h) && ok16(a.mixes) && ok16(a.mu);
        const int units = vec ? a.W / 8 : a.W;
        const dim3 grid(a.T, a.T >= 256 ? 1 : (units + 255) / 256);      // few rows: a block per 256 accesses of a row
        if (vec) tb_launch(wkv_shift_kernel<T, true>, grid, 256, 0, stream, a);
        else tb_launch(wkv_shift_kernel<T, false>, grid, 256, 0, stream, a);
    }
    else if (stage == 1) tb_launch(wkv_decay_kernel<T>, dim3((a.T + DEC_TOK - 1) / DEC_TOK, (a.H * a.dk + 127) / 128), 128, 0, stream, a);
    else if (stage == 2) {
        // eight lanes a column while four would leave SMs without a block (148 on this chip), for heads up to 128 wide
        const bool few = (long long)a.B * a.H * ((a.dk + 31) / 32) < 148 && a.dk <= 128;
        if (few) {
            if (a.dk <= 32) launch_scan<T, 4, 16, 8>(a, stream);
            else if (a.dk <= 64) launch_scan<T, 8, 16, 8>(a, stream);
            else launch_scan<T, 16, 16, 8>(a, stream);
        } else if (a.dk <= 32) launch_scan<T, 8, 16, 4>(a, stream);
        else if (a.dk <= 64) launch_scan<T, 16, 16, 4>(a, stream);
        else if (a.dk <= 128) launch_scan<T, 32, 8, 4>(a, stream);
        else launch_scan<T, 64, 8, 4>(a, stream);
    } else tb_launch(wkv_out_kernel<T>, dim3(a.T, (a.H + 3) / 4), 128, 0, stream, a);
    return 0;
}

}  // namespace

// stage 0: the mixes; 1: the decay; 2: the recurrence; 3: unit norm, weight and gate.
extern "C" int tb_wkv(const WkvArgs* args, int stage, int dtype, cudaStream_t stream) {
    WkvArgs a = *args;
    TB_REQUIRE(stage >= 0 && stage <= 3, "wkv: unknown stage %d", stage);
    TB_REQUIRE(a.T > 0 && a.B > 0 && a.H > 0 && a.dk > 0 && a.W > 0, "wkv: sizes must be positive");
    TB_REQUIRE(a.dk <= 256, "wkv: %d key channels a head (at most 256)", a.dk);
    TB_REQUIRE(a.H <= 65535 && a.T <= 2147483647, "wkv: too many heads");
    TB_REQUIRE(a.state && a.state_stride >= (long long)a.H * a.dk * a.dk + a.W, "wkv: the state row is shorter than the heads' states and an input row");
    TB_REQUIRE(stage != 0 || (a.h && a.mixes && a.mu && a.seq_of && a.q_start && a.slot_of_seq), "wkv: the mixes need rows, factors and the layout");
    TB_REQUIRE(stage != 1 || (a.lora && a.w2 && a.w0 && a.decay && a.rank > 0 && a.rank <= 8192), "wkv: the decay needs its low-rank row and matrices");
    TB_REQUIRE(stage != 2 || (a.h && a.proj && a.decay && a.u && a.out && a.q_start && a.slot_of_seq), "wkv: the recurrence needs projections, decay, bonus and the layout");
    TB_REQUIRE(stage != 3 || (a.out && a.proj && a.norm_w && a.y), "wkv: the output step needs sums, gate, weight and a place for the result");
    if (dtype == TB_F32) run<float>(a, stage, stream);
    else if (dtype == TB_BF16) run<__nv_bfloat16>(a, stage, stream);
    else TB_REQUIRE(false, "wkv: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("wkv");
    return 0;
}
