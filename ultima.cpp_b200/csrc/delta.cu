// The gated delta-rule mixer: a recurrent layer whose state is, for every head, a matrix S [D, E]
// (D key channels, E value channels) in float32, plus the last inputs of a short causal convolution.
//
// For one token of one head, with unit vectors q (scaled) and k, a value v, a write strength b in
// (0, 1) and a decay a[d] in (0, 1) for every key channel:
//     S[d, :] *= a[d];   u = b * (v - S^T k);   S += k u^T;   o = S^T q
// so the read-out sees the token's own write.  Every column of S evolves on its own, which is what
// the scan kernel uses: a group of eight lanes holds one column, tokens are taken in order.
//
// Four kernels, for prompts and single tokens alike (a step's tokens of one sequence are rows
// seq_start[s] .. seq_start[s + 1] of the packed batch; state rows are slot numbers):
//   delta_prepare      short convolution + SiLU of q, k, v; unit vectors; write strength; decay
//   conv_state_update  the convolution's last inputs, carried to the next step
//   delta_scan         the recurrence
//   delta_finish       per-head RMS norm of o, weight, sigmoid output gate from a low-rank product
// Everything is float32; the projections come in as float32 sums of the products.
#include "common.cuh"

constexpr int MAX_TAPS = 16;
constexpr int MAX_RANK = 256;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct DeltaShape {
    int H, G, D, E;          // heads, q/k heads, key size, value size
    int taps;                // convolution length (the last tap is the current token's)
    int rank_a, rank_g;      // inner sizes of the decay's and the gate's low-rank products
    int q_off, k_off, v_off, b_off, a_off, g_off;   // columns of a projection row
    long long ldp;           // row stride of the projections
};

// One warp a (token, unit); units of a token: G query heads, G key heads, H value heads (which also
// make the head's write strength and decay).
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float* __restrict__ p, DeltaShape s, const float* __restrict__ conv_w,
                     const float* __restrict__ conv_state, const float* __restrict__ a2,
                     const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                     const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                     const int* __restrict__ seq_slot, float* __restrict__ qn, float* __restrict__ kn,
                     float* __restrict__ vc, float* __restrict__ beta, float* __restrict__ dec,
                     int n_tokens, float unit_eps, float q_scale) {
    pdl_trigger();
    pdl_wait();
    const int units = 2 * s.G + s.H;
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)n_tokens * units) return;
    const int t = (int)(wid / units), unit = (int)(wid % units);
    const int seq = tok_seq[t];
    const int r = t - seq_start[seq];
    const int K = s.taps - 1;
    const int C = 2 * s.G * s.D + s.H * s.E;
    const float* st = conv_state + (long long)seq_slot[seq] * K * C;

    auto conv_silu = [&](int c) -> float {
        float acc = 0.f;
        for (int j = K; j >= 0; --j) {                 // oldest input first
            const float w = conv_w[(long long)c * s.taps + (s.taps - 1 - j)];
            const float x = (r - j >= 0) ? p[(long long)(t - j) * s.ldp + c] : st[(long long)(K + r - j) * C + c];
            acc = fmaf(w, x, acc);
        }
        return acc * sigmoidf_(acc);
    };

    if (unit < 2 * s.G) {
        const bool is_q = unit < s.G;
        const int head = is_q ? unit : unit - s.G;
        const int c0 = (is_q ? s.q_off : s.k_off) + head * s.D;      // q_off = 0 and k_off = G * D: columns are channels
        float vals[8];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            vals[i] = d < s.D ? conv_silu(c0 + d) : 0.f;
            ss += vals[i] * vals[i];
        }
        ss = warp_sum(ss);
        const float inv = (is_q ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
        float* o = (is_q ? qn : kn) + (long long)t * s.G * s.D + head * s.D;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            if (d < s.D) o[d] = vals[i] * inv;
        }
        return;
    }
    const int h = unit - 2 * s.G;
    for (int e = lane; e < s.E; e += 32)
        vc[(long long)t * s.H * s.E + h * s.E + e] = conv_silu(s.v_off + h * s.E + e);
    const float* row = p + (long long)t * s.ldp;
    if (lane == 0) beta[(long long)t * s.H + h] = sigmoidf_(row[s.b_off + h]);
    const float rate = expf(a_log[h]);
    for (int d = lane; d < s.D; d += 32) {
        const int c = h * s.D + d;
        float a = dt_bias[c];
        for (int k = 0; k < s.rank_a; ++k) a = fmaf(a2[(long long)c * s.rank_a + k], row[s.a_off + k], a);
        dec[(long long)t * s.H * s.D + c] = expf(-rate * softplusf_(a));
    }
}

// One thread a (sequence, channel): the last taps - 1 inputs of what the state held followed by the step's.
__global__ void conv_state_update_kernel(const float* __restrict__ p, long long ldp, float* __restrict__ conv_state,
                                         const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                                         int n_seqs, int C, int taps) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_seqs * C) return;
    const int b = (int)(i / C), c = (int)(i % C);
    const int K = taps - 1;
    const int first = seq_start[b], n = seq_start[b + 1] - first;
    float* st = conv_state + (long long)seq_slot[b] * K * C;
    float tmp[MAX_TAPS];
    for (int k = 0; k < K; ++k) {
        const int rel = n - K + k;
        tmp[k] = rel >= 0 ? p[(long long)(first + rel) * ldp + c] : st[(long long)(K + rel) * C + c];
    }
    for (int k = 0; k < K; ++k) st[(long long)k * C + c] = tmp[k];
}

// The recurrence.  A block takes 32 value channels of one head of one sequence; eight lanes hold one
// column of S (lane p the key channels p, p + 8, ...), so a warp holds four columns and a dot product
// over the key channels ends in three exchanges.  Tokens come through shared memory eight at a time.
constexpr int SCAN_COLS = 32, SCAN_LANES = 8, SCAN_TOKENS = 8;

template <int R>
__global__ void __launch_bounds__(SCAN_COLS * SCAN_LANES)
delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vc,
                  const float* __restrict__ beta, const float* __restrict__ dec, float* __restrict__ out,
                  float* __restrict__ S, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                  int H, int G, int D, int E) {
    constexpr int DP = SCAN_LANES * R;
    __shared__ float sq[SCAN_TOKENS][DP], sk[SCAN_TOKENS][DP], sa[SCAN_TOKENS][DP];
    __shared__ float sv[SCAN_TOKENS][SCAN_COLS], sb[SCAN_TOKENS];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x;
    const int col = tid / SCAN_LANES, p = tid % SCAN_LANES;
    const int h = blockIdx.y, b = blockIdx.z;
    const int g = h / (H / G);
    const int j = blockIdx.x * SCAN_COLS + col;
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    if (t0 >= t1) return;
    float* Sh = S + ((long long)seq_slot[b] * H + h) * D * E;
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = p + SCAN_LANES * i;
        s[i] = (d < D && j < E) ? Sh[(long long)d * E + j] : 0.f;
    }
    for (int base = t0; base < t1; base += SCAN_TOKENS) {
        const int n = min(SCAN_TOKENS, t1 - base);
        __syncthreads();
        for (int idx = tid; idx < n * DP; idx += blockDim.x) {
            const int tt = idx / DP, d = idx % DP;
            const long long t = base + tt;
            const bool in = d < D;
            sq[tt][d] = in ? qn[(t * G + g) * D + d] : 0.f;
            sk[tt][d] = in ? kn[(t * G + g) * D + d] : 0.f;
            sa[tt][d] = in ? dec[(t * H + h) * D + d] : 1.f;
        }
        for (int idx = tid; idx < n * SCAN_COLS; idx += blockDim.x) {
            const int tt = idx / SCAN_COLS, c = idx % SCAN_COLS;
            const int jj = blockIdx.x * SCAN_COLS + c;
            sv[tt][c] = jj < E ? vc[((long long)(base + tt) * H + h) * E + jj] : 0.f;
        }
        if (tid < n) sb[tid] = beta[(long long)(base + tid) * H + h];
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const int d = p + SCAN_LANES * i;
                s[i] *= sa[tt][d];
                dot = fmaf(s[i], sk[tt][d], dot);
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            const float u = sb[tt] * (sv[tt][col] - dot);
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const int d = p + SCAN_LANES * i;
                s[i] = fmaf(sk[tt][d], u, s[i]);
                o = fmaf(s[i], sq[tt][d], o);
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (p == 0 && j < E) out[((long long)(base + tt) * H + h) * E + j] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = p + SCAN_LANES * i;
        if (d < D && j < E) Sh[(long long)d * E + j] = s[i];
    }
}

// One warp a (token, head): o / rms(o) * w * sigmoid(g2 (g1 h)), g1 h being columns of the projection row.
template <typename TO>
__global__ void __launch_bounds__(128)
delta_finish_kernel(const float* __restrict__ o, const float* __restrict__ p, long long ldp, int g_off, int rank_g,
                    const float* __restrict__ g2, const float* __restrict__ w, TO* __restrict__ out,
                    int n_tokens, int H, int E, float eps) {
    pdl_trigger();
    pdl_wait();
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)n_tokens * H) return;
    const long long t = wid / H;
    const int h = (int)(wid % H);
    const float* orow = o + (t * H + h) * E;
    float ss = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = orow[e]; ss += v * v; }
    ss = warp_sum(ss);
    const float inv = inv_rms(ss, (float)E, eps);
    const float* low = p + t * ldp + g_off;
    for (int e = lane; e < E; e += 32) {
        const int c = h * E + e;
        float z = 0.f;
        for (int k = 0; k < rank_g; ++k) z = fmaf(g2[(long long)c * rank_g + k], low[k], z);
        out[(t * H + h) * E + e] = from_f32<TO>(orow[e] * inv * w[e] * sigmoidf_(z));
    }
}

// ---------------------------------------------------------------------------------------
// shape: [H, G, D, E, taps, rank_a, rank_g, q_off, k_off, v_off, b_off, a_off, g_off] (13 ints)
static int read_shape(const int* shape, long long ldp, DeltaShape& s) {
    s.H = shape[0]; s.G = shape[1]; s.D = shape[2]; s.E = shape[3]; s.taps = shape[4];
    s.rank_a = shape[5]; s.rank_g = shape[6];
    s.q_off = shape[7]; s.k_off = shape[8]; s.v_off = shape[9]; s.b_off = shape[10]; s.a_off = shape[11]; s.g_off = shape[12];
    s.ldp = ldp;
    if (s.H <= 0 || s.G <= 0 || s.H % s.G || s.D <= 0 || s.D > 256 || s.E <= 0 || s.taps < 1 || s.taps > MAX_TAPS ||
        s.rank_a < 1 || s.rank_a > MAX_RANK || s.rank_g < 1 || s.rank_g > MAX_RANK || s.H > 65535) return UB_ERR_ARG;
    // the convolution's state is indexed by projection column: q, k, v are the row's first columns
    if (s.q_off != 0 || s.k_off != s.G * s.D || s.v_off != 2 * s.G * s.D) return UB_ERR_ARG;
    return 0;
}

UB_API int ub_delta_prepare(const float* p, long long ldp, const int* shape, const float* conv_w, const float* conv_state,
                            const float* a2, const float* dt_bias, const float* a_log, const int* tok_seq,
                            const int* seq_start, const int* seq_slot, float* qn, float* kn, float* vc, float* beta,
                            float* dec, int n_tokens, float unit_eps, float q_scale, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    DeltaShape s;
    if (int rc = read_shape(shape, ldp, s)) return rc;
    const long long warps = (long long)n_tokens * (2 * s.G + s.H);
    const unsigned grid = (unsigned)((warps + 3) / 4);
    return (int)ub_launch_dependent(delta_prepare_kernel, dim3(grid), dim3(128), 0, st, p, s, conv_w, conv_state, a2, dt_bias,
                                    a_log, tok_seq, seq_start, seq_slot, qn, kn, vc, beta, dec, n_tokens, unit_eps, q_scale);
}

UB_API int ub_conv_state_update(const float* p, long long ldp, float* conv_state, const int* seq_start, const int* seq_slot,
                                int n_seqs, int C, int taps, cudaStream_t st) {
    if (n_seqs <= 0 || taps <= 1) return 0;
    if (taps > MAX_TAPS) return UB_ERR_ARG;
    const long long n = (long long)n_seqs * C;
    return (int)ub_launch_dependent(conv_state_update_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, st, p, ldp,
                                    conv_state, seq_start, seq_slot, n_seqs, C, taps);
}

UB_API int ub_delta_scan(const float* qn, const float* kn, const float* vc, const float* beta, const float* dec, float* out,
                         float* S, const int* seq_start, const int* seq_slot, int n_seqs, int H, int G, int D, int E,
                         cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || D > 256 || E <= 0 || H > 65535 || n_seqs > 65535) return UB_ERR_ARG;
    const dim3 grid((E + SCAN_COLS - 1) / SCAN_COLS, H, n_seqs), block(SCAN_COLS * SCAN_LANES);
    cudaError_t e;
#define GO(R) e = ub_launch_dependent(delta_scan_kernel<R>, grid, block, 0, st, qn, kn, vc, beta, dec, out, S, seq_start, seq_slot, H, G, D, E)
    if (D <= 16) GO(2);
    else if (D <= 32) GO(4);
    else if (D <= 64) GO(8);
    else if (D <= 128) GO(16);
    else GO(32);
#undef GO
    return (int)e;
}

UB_API int ub_delta_finish(const float* o, const float* p, long long ldp, int g_off, int rank_g, const float* g2,
                           const float* w, void* out, int out_dtype, int n_tokens, int H, int E, float eps, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (rank_g < 1 || rank_g > MAX_RANK) return UB_ERR_ARG;
    const long long warps = (long long)n_tokens * H;
    const unsigned grid = (unsigned)((warps + 3) / 4);
    cudaError_t e;
    if (out_dtype == UB_F32)
        e = ub_launch_dependent(delta_finish_kernel<float>, dim3(grid), dim3(128), 0, st, o, p, ldp, g_off, rank_g, g2, w, (float*)out, n_tokens, H, E, eps);
    else if (out_dtype == UB_BF16)
        e = ub_launch_dependent(delta_finish_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, st, o, p, ldp, g_off, rank_g, g2, w, (__nv_bfloat16*)out, n_tokens, H, E, eps);
    else return UB_ERR_UNSUPPORTED;
    return (int)e;
}
