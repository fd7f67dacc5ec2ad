// Layers that carry a state of fixed size from token to token: a short causal convolution over time, and the
// gated linear recurrence  S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t  (S is K x V per head, float).
//
// Two ways of forming a_t, k_t, q_t, v_t from a layer's projections are built:
//   "ssd"  (a state-space layer with a scalar decay a head): a = exp(-exp(A_log) dt), dt = softplus(raw + bias),
//          k = dt * B, q = C (B and C shared by the heads of a group), v = x, and o += D x;
//   "gate" (linear attention whose forget gate also decides what is written): a = f, k = 1 - f,
//          f = low + (1 - low) sigmoid(raw + bias) per head and channel, q = silu(raw q).
// Everything after the projections (step sizes, decays, gates, the state, the sums) is float; results leave as float and
// are normed by group_rmsnorm_kernel, which rounds once.  A sequence's tokens are taken in order, one after another,
// with the same arithmetic for every token, so results do not depend on how a prompt is cut into steps.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------------------------------------------------------------
// Causal convolution over time on each channel:  y_t = act(bias + sum_j w[c, j] x_(t - taps + 1 + j)) (+ x_t).
// The last taps - 1 inputs of every sequence live in `ring` [slots, taps - 1, channels], input p at row p % (taps - 1).
// Inputs of the step's own tokens come from `x`, older ones from the ring, positions below 0 are zero.
// write_state: a thread whose token is among the last taps - 1 of its sequence's portion stores its input.  That is
// safe inside this kernel only when no other thread reads the row it overwrites, which holds when every sequence
// brings one token (the row it overwrites is the oldest one it read itself); otherwise the state is written by
// short_conv_state_kernel afterwards.
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ x, int ld_x, const float* __restrict__ w, const float* __restrict__ bias,
                                  T* __restrict__ out, int ld_out, T* __restrict__ ring, int channels, int taps,
                                  const int* __restrict__ positions, const int* __restrict__ seq_index,
                                  const int* __restrict__ slots, const int* __restrict__ q_start, size_t total, int act,
                                  int residual, int write_state) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int t = (int)(idx / channels), c = (int)(idx - (size_t)t * channels);
    const int seq = seq_index[t], pos = positions[t];
    const int i = t - q_start[seq];
    const int keep = taps - 1;
    T* rows = ring + (size_t)slots[seq] * (keep > 0 ? keep : 1) * channels;
    const float cur = to_float(x[(size_t)t * ld_x + c]);
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = keep - j, p = pos - back;
        float v;
        if (back == 0) v = cur;
        else if (p < 0) v = 0.f;
        else if (back <= i) v = to_float(x[(size_t)(t - back) * ld_x + c]);
        else v = to_float(rows[(size_t)(p % keep) * channels + c]);
        acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    if (act == 1) acc = siluf_(acc);
    if (residual) acc += cur;
    out[(size_t)t * ld_out + c] = from_float<T>(acc);
    if (write_state && keep > 0 && q_start[seq + 1] - 1 - t < keep) rows[(size_t)(pos % keep) * channels + c] = x[(size_t)t * ld_x + c];
}

// The inputs of the last taps - 1 tokens of every sequence's portion go into the ring (after the kernel above has read it).
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ x, int ld_x, T* __restrict__ ring, int channels, int keep,
                                        const int* __restrict__ positions, const int* __restrict__ slots,
                                        const int* __restrict__ q_start, int n_seqs) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_seqs * keep * channels) return;
    const int c = (int)(idx % channels);
    const int r = (int)((idx / channels) % keep);
    const int seq = (int)(idx / ((size_t)channels * keep));
    const int t = q_start[seq + 1] - 1 - r;
    if (t < q_start[seq]) return;
    T* rows = ring + (size_t)slots[seq] * keep * channels;
    rows[(size_t)(positions[t] % keep) * channels + c] = x[(size_t)t * ld_x + c];
}

// ---------------------------------------------------------------------------------------------------------------------
// The recurrence.  A warp owns 8 columns (v) of a head's state; the K rows of a column are shared by 4 lanes (lane =
// part * 8 + column; a lane holds KPT consecutive rows), so loading and storing the state touches whole 32-byte sectors
// and a token's output needs two shuffles.  A block has blockDim.x / 32 warps on neighbouring columns of one head of one
// sequence; grid (column tiles, heads, sequences).  The step's a, k, q, v are formed in float by the whole block, STEPS
// tokens at a time, into shared memory; the warps then run those tokens without meeting.
constexpr int REC_COLS = 8, REC_PARTS = 4;
enum { REC_SSD = 0, REC_GATE = 1 };

struct RecurrenceArgs {
    float* state;           // [slots, heads, K, V]
    float* out;             // [tokens, heads * V]
    const int* q_start;
    const int* slots;
    int heads, K, V, steps;
    // ssd: conv = rows [x (heads * V) | B (groups * K) | C (groups * K)], dt = a column block of the input projection
    // gate: q, f, v = column blocks of the projection
    const void* a0; int ld0;    // ssd: conv rows            gate: q
    const void* a1; int ld1;    // ssd: dt                   gate: f
    const void* a2; int ld2;    // ssd: -                    gate: v
    const float* p0;            // ssd: dt bias [heads]      gate: f bias [heads * K]
    const float* p1;            // ssd: A_log [heads]        gate: lower bound [heads * K]
    const float* p2;            // ssd: D [heads]
    int groups;                 // ssd: groups of heads that share B and C
};

template <typename T, int KPT, int MODE>
__global__ void __launch_bounds__(256) linear_recurrence_kernel(const RecurrenceArgs A) {
    extern __shared__ __align__(16) float rec_smem[];
    allow_dependents();
    wait_for_prior_kernels();
    constexpr int KROW = REC_PARTS * (KPT + 4);     // a lane's KPT numbers, 4 floats of padding between lanes' runs
    const int warps = blockDim.x >> 5, cols = warps * REC_COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int part = lane >> 3, col8 = lane & 7;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int v0 = blockIdx.x * cols;
    const int vcol = v0 + warp * REC_COLS + col8;
    const bool v_ok = vcol < A.V;
    const int t0 = A.q_start[seq], t1 = A.q_start[seq + 1];
    const int K = A.K, V = A.V, H = A.heads, STEPS = A.steps;
    float* qs = rec_smem;                        // [STEPS][KROW]
    float* ks = qs + STEPS * KROW;               // [STEPS][KROW]
    float* as = ks + STEPS * KROW;               // gate: [STEPS][KROW]; ssd: [STEPS]
    float* vs = as + (MODE == REC_GATE ? STEPS * KROW : STEPS);   // [STEPS][cols]
    float* sbase = A.state + ((size_t)A.slots[seq] * H + h) * K * V;

    float S[KPT];
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const int k = part * KPT + i;
        S[i] = (v_ok && k < K) ? sbase[(size_t)k * V + vcol] : 0.f;
    }
    const float skip = (MODE == REC_SSD && A.p2) ? A.p2[h] : 0.f;

    for (int ts = t0; ts < t1; ts += STEPS) {
        const int ns = min(STEPS, t1 - ts);
        __syncthreads();
        // ---- the block forms the tokens' a, k, q, v
        if (MODE == REC_SSD) {
            const T* conv = (const T*)A.a0;
            const T* dtp = (const T*)A.a1;
            const int g = h / (H / A.groups);
            const int b_off = H * V + g * K, c_off = H * V + A.groups * K + g * K;
            for (int e = threadIdx.x; e < ns * REC_PARTS * KPT; e += blockDim.x) {
                const int s = e / (REC_PARTS * KPT), k = e - s * (REC_PARTS * KPT);
                const int t = ts + s;
                const float dt = softplusf_(to_float(dtp[(size_t)t * A.ld1 + h]) + A.p0[h]);
                const int at = s * KROW + (k / KPT) * (KPT + 4) + k % KPT;
                float kb = 0.f, qc = 0.f;
                if (k < K) {
                    kb = dt * to_float(conv[(size_t)t * A.ld0 + b_off + k]);
                    qc = to_float(conv[(size_t)t * A.ld0 + c_off + k]);
                }
                ks[at] = kb;
                qs[at] = qc;
                if (k == 0) as[s] = expf(-expf(A.p1[h]) * dt);
            }
            for (int e = threadIdx.x; e < ns * cols; e += blockDim.x) {
                const int s = e / cols, j = e - s * cols;
                vs[s * cols + j] = (v0 + j < V) ? to_float(conv[(size_t)(ts + s) * A.ld0 + h * V + v0 + j]) : 0.f;
            }
        } else {
            const T* qp = (const T*)A.a0;
            const T* fp = (const T*)A.a1;
            const T* vp = (const T*)A.a2;
            for (int e = threadIdx.x; e < ns * REC_PARTS * KPT; e += blockDim.x) {
                const int s = e / (REC_PARTS * KPT), k = e - s * (REC_PARTS * KPT);
                const int t = ts + s;
                const int at = s * KROW + (k / KPT) * (KPT + 4) + k % KPT;
                float f = 0.f, q = 0.f, w = 0.f;
                if (k < K) {
                    const float low = A.p1[h * K + k];
                    f = low + (1.f - low) * sigmoidf_(to_float(fp[(size_t)t * A.ld1 + h * K + k]) + A.p0[h * K + k]);
                    w = 1.f - f;
                    q = siluf_(to_float(qp[(size_t)t * A.ld0 + h * K + k]));
                }
                as[at] = f;
                ks[at] = w;
                qs[at] = q;
            }
            for (int e = threadIdx.x; e < ns * cols; e += blockDim.x) {
                const int s = e / cols, j = e - s * cols;
                vs[s * cols + j] = (v0 + j < V) ? to_float(vp[(size_t)(ts + s) * A.ld2 + h * V + v0 + j]) : 0.f;
            }
        }
        __syncthreads();
        // ---- each warp runs the tokens on its columns
        for (int s = 0; s < ns; ++s) {
            const float v = vs[s * cols + warp * REC_COLS + col8];
            const float* qrow = qs + s * KROW + part * (KPT + 4);
            const float* krow = ks + s * KROW + part * (KPT + 4);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            if (MODE == REC_SSD) {
                const float a = as[s];
#pragma unroll
                for (int i = 0; i < KPT; i += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(krow + i);
                    const float4 q4 = *reinterpret_cast<const float4*>(qrow + i);
                    S[i] = fmaf(a, S[i], k4.x * v);         acc[0] = fmaf(S[i], q4.x, acc[0]);
                    S[i + 1] = fmaf(a, S[i + 1], k4.y * v); acc[1] = fmaf(S[i + 1], q4.y, acc[1]);
                    S[i + 2] = fmaf(a, S[i + 2], k4.z * v); acc[2] = fmaf(S[i + 2], q4.z, acc[2]);
                    S[i + 3] = fmaf(a, S[i + 3], k4.w * v); acc[3] = fmaf(S[i + 3], q4.w, acc[3]);
                }
            } else {
                const float* arow = as + s * KROW + part * (KPT + 4);
#pragma unroll
                for (int i = 0; i < KPT; i += 4) {
                    const float4 a4 = *reinterpret_cast<const float4*>(arow + i);
                    const float4 k4 = *reinterpret_cast<const float4*>(krow + i);
                    const float4 q4 = *reinterpret_cast<const float4*>(qrow + i);
                    S[i] = fmaf(a4.x, S[i], k4.x * v);         acc[0] = fmaf(S[i], q4.x, acc[0]);
                    S[i + 1] = fmaf(a4.y, S[i + 1], k4.y * v); acc[1] = fmaf(S[i + 1], q4.y, acc[1]);
                    S[i + 2] = fmaf(a4.z, S[i + 2], k4.z * v); acc[2] = fmaf(S[i + 2], q4.z, acc[2]);
                    S[i + 3] = fmaf(a4.w, S[i + 3], k4.w * v); acc[3] = fmaf(S[i + 3], q4.w, acc[3]);
                }
            }
            float o = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            o += __shfl_xor_sync(0xffffffffu, o, 8);
            o += __shfl_xor_sync(0xffffffffu, o, 16);
            if (part == 0 && v_ok) A.out[((size_t)(ts + s) * H + h) * V + vcol] = fmaf(skip, v, o);
        }
    }
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const int k = part * KPT + i;
        if (v_ok && k < K) sbase[(size_t)k * V + vcol] = S[i];
    }
}

// out[t, g, :] = u / sqrt(mean(u^2) + eps) * w,  u = y[t, g, :] (* act(gate[t, g, :])): an RMS norm on each of a row's
// groups, the optional gate applied BEFORE the norm.  y is float; the weight has `period` numbers and repeats (a weight
// of one group's size is shared by all groups).  One block a (token, group).  out_scale multiplies the result before it is
// rounded.
template <typename T>
__global__ void group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int ld_gate, const float* __restrict__ w,
                                     int period, float eps, T* __restrict__ out, int ld_out, int groups, int size, float out_scale) {
    __shared__ float scratch[32];
    allow_dependents();
    wait_for_prior_kernels();
    const int t = blockIdx.x / groups, g = blockIdx.x - t * groups;
    const float* row = y + ((size_t)t * groups + g) * size;
    const T* grow = gate ? gate + (size_t)t * ld_gate + (size_t)g * size : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float u = row[i];
        if (grow) u *= siluf_(to_float(grow[i]));
        ss += u * u;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float u = row[i];
        if (grow) u *= siluf_(to_float(grow[i]));
        out[(size_t)t * ld_out + (size_t)g * size + i] = from_float<T>(u * inv * w[(g * size + i) % period] * out_scale);
    }
}

// out[t, h, 0:vdim] = o[t, h, 0:vdim] * sigmoid(gate[t, h * vdim + d]); o's heads are `o_head` numbers apart (heads
// padded to a wider size keep their first vdim numbers), out is dense.  out may be o when o_head == vdim.
template <typename T>
__global__ void sigmoid_gate_kernel(const T* o, int o_head, const T* __restrict__ gate, int ld_gate, T* out, int heads, int vdim,
                                    size_t total) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t per_row = (size_t)heads * vdim;
    const size_t t = idx / per_row;
    const int r = (int)(idx - t * per_row);
    const int h = r / vdim, d = r - h * vdim;
    const float v = to_float(o[(t * heads + h) * o_head + d]);
    out[idx] = from_float<T>(v * sigmoidf_(to_float(gate[t * ld_gate + r])));
}

template <typename T, int MODE>
int launch_recurrence(const RecurrenceArgs& a, int n_seqs, int warps, cudaStream_t s) {
    const int cols = warps * REC_COLS;
    dim3 grid((a.V + cols - 1) / cols, a.heads, n_seqs), block(warps * 32);
    RecurrenceArgs args = a;
    auto smem_of = [&](int kpt, int steps) {
        const int krow = REC_PARTS * (kpt + 4);
        return (size_t)(steps * krow * 2 + (MODE == REC_GATE ? steps * krow : steps) + steps * cols) * sizeof(float);
    };
#define RMX_REC_CASE(KPT, STEPS)                                                                                           \
    do {                                                                                                                   \
        args.steps = STEPS;                                                                                                \
        RMX_CHECK_LAUNCHED(launch_dependent(linear_recurrence_kernel<T, KPT, MODE>, grid, block, smem_of(KPT, STEPS), s, args), \
                           "linear_recurrence");                                                                           \
        return 0;                                                                                                          \
    } while (0)
    if (a.K <= 32) RMX_REC_CASE(8, 16);
    if (a.K <= 64) RMX_REC_CASE(16, 16);
    if (a.K <= 128) RMX_REC_CASE(32, 8);
    if (a.K <= 256) RMX_REC_CASE(64, 4);
#undef RMX_REC_CASE
    RMX_FAIL("linear_recurrence: a state of %d rows a head is beyond 256", a.K);
}
}  // namespace

RMX_API int rmx_short_conv(const void* x, int ld_x, const float* w, const float* bias, void* out, int ld_out, void* ring, int channels,
                           int taps, const int* positions, const int* seq_index, const int* slots, const int* q_start, int n_tokens,
                           int n_seqs, int act, int residual, int single_tokens, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && n_seqs > 0 && channels > 0 && taps >= 1 && ld_x >= channels && ld_out >= channels, "short_conv: bad sizes");
    RMX_REQUIRE(x && w && out && ring && positions && seq_index && slots && q_start, "short_conv: a null pointer");
    RMX_REQUIRE(act == 0 || act == 1, "short_conv: unknown activation %d", act);
    const size_t total = (size_t)n_tokens * channels;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    const int keep = taps - 1;
    const size_t state_items = (size_t)n_seqs * keep * channels;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32) {
        RMX_CHECK_LAUNCHED(launch_dependent(short_conv_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)x, ld_x, w, bias, (float*)out,
                                            ld_out, (float*)ring, channels, taps, positions, seq_index, slots, q_start, total, act, residual,
                                            single_tokens), "short_conv");
        if (!single_tokens && keep > 0)
            RMX_CHECK_LAUNCHED(launch_dependent(short_conv_state_kernel<float>, dim3((unsigned)((state_items + threads - 1) / threads)), dim3(threads),
                                                0, s, (const float*)x, ld_x, (float*)ring, channels, keep, positions, slots, q_start, n_seqs),
                               "short_conv_state");
    } else if (dtype == RMX_BF16) {
        RMX_CHECK_LAUNCHED(launch_dependent(short_conv_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)x, ld_x, w,
                                            bias, (__nv_bfloat16*)out, ld_out, (__nv_bfloat16*)ring, channels, taps, positions, seq_index, slots,
                                            q_start, total, act, residual, single_tokens), "short_conv");
        if (!single_tokens && keep > 0)
            RMX_CHECK_LAUNCHED(launch_dependent(short_conv_state_kernel<__nv_bfloat16>, dim3((unsigned)((state_items + threads - 1) / threads)),
                                                dim3(threads), 0, s, (const __nv_bfloat16*)x, ld_x, (__nv_bfloat16*)ring, channels, keep, positions,
                                                slots, q_start, n_seqs), "short_conv_state");
    } else {
        RMX_FAIL("short_conv: unknown dtype %d", dtype);
    }
    return 0;
}

// mode 0 ("ssd"): a0 = conv rows [x | B | C], a1 = dt columns, p0 = dt bias, p1 = A_log, p2 = D (or null), groups.
// mode 1 ("gate"): a0 = q, a1 = f, a2 = v columns, p0 = f bias, p1 = lower bound.
RMX_API int rmx_linear_recurrence(int mode, float* state, float* out, const int* q_start, const int* slots, int n_seqs, int heads, int K,
                                  int V, const void* a0, int ld0, const void* a1, int ld1, const void* a2, int ld2, const float* p0,
                                  const float* p1, const float* p2, int groups, int warps, int dtype, void* stream) {
    if (n_seqs == 0) return 0;
    RMX_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && heads > 0 && heads <= 65535 && K > 0 && V > 0, "linear_recurrence: bad sizes");
    RMX_REQUIRE(state && out && q_start && slots && a0 && a1 && p0 && p1, "linear_recurrence: a null pointer");
    RMX_REQUIRE(warps >= 1 && warps <= 8, "linear_recurrence: 1 to 8 warps a block");
    RecurrenceArgs a;
    a.state = state; a.out = out; a.q_start = q_start; a.slots = slots;
    a.heads = heads; a.K = K; a.V = V; a.steps = 0;
    a.a0 = a0; a.ld0 = ld0; a.a1 = a1; a.ld1 = ld1; a.a2 = a2; a.ld2 = ld2;
    a.p0 = p0; a.p1 = p1; a.p2 = p2; a.groups = groups;
    cudaStream_t s = (cudaStream_t)stream;
    if (mode == REC_SSD) {
        RMX_REQUIRE(groups > 0 && heads % groups == 0, "linear_recurrence: %d heads in %d groups", heads, groups);
        if (dtype == RMX_F32) return launch_recurrence<float, REC_SSD>(a, n_seqs, warps, s);
        if (dtype == RMX_BF16) return launch_recurrence<__nv_bfloat16, REC_SSD>(a, n_seqs, warps, s);
    } else if (mode == REC_GATE) {
        RMX_REQUIRE(a2 != nullptr, "linear_recurrence: the gated form needs values");
        if (dtype == RMX_F32) return launch_recurrence<float, REC_GATE>(a, n_seqs, warps, s);
        if (dtype == RMX_BF16) return launch_recurrence<__nv_bfloat16, REC_GATE>(a, n_seqs, warps, s);
    } else {
        RMX_FAIL("linear_recurrence: unknown mode %d", mode);
    }
    RMX_FAIL("linear_recurrence: unknown dtype %d", dtype);
}

RMX_API int rmx_group_rmsnorm(const float* y, const void* gate, int ld_gate, const float* w, int period, float eps, void* out, int ld_out,
                              int n_tokens, int groups, int size, float out_scale, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && groups > 0 && size > 0 && period > 0 && y && w && out, "group_rmsnorm: bad sizes or a null pointer");
    RMX_REQUIRE((long long)n_tokens * groups < (1LL << 31), "group_rmsnorm: too many groups");
    int threads = (size + 31) / 32 * 32;
    threads = threads > 256 ? 256 : threads;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((unsigned)(n_tokens * groups));
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(group_rmsnorm_kernel<float>, grid, dim3(threads), 0, s, y, (const float*)gate, ld_gate, w, period, eps,
                                            (float*)out, ld_out, groups, size, out_scale), "group_rmsnorm");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(group_rmsnorm_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, y, (const __nv_bfloat16*)gate, ld_gate,
                                            w, period, eps, (__nv_bfloat16*)out, ld_out, groups, size, out_scale), "group_rmsnorm");
    else
        RMX_FAIL("group_rmsnorm: unknown dtype %d", dtype);
    return 0;
}

RMX_API int rmx_sigmoid_gate(const void* o, int o_head, const void* gate, int ld_gate, void* out, int n_tokens, int heads, int vdim,
                             int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && heads > 0 && vdim > 0 && o_head >= vdim && ld_gate >= heads * vdim && o && gate && out,
                "sigmoid_gate: bad sizes or a null pointer");
    RMX_REQUIRE(o != out || o_head == vdim, "sigmoid_gate: in place only where heads are not padded");
    const size_t total = (size_t)n_tokens * heads * vdim;
    const int threads = 256;
    const dim3 grid((unsigned)((total + threads - 1) / threads));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(sigmoid_gate_kernel<float>, grid, dim3(threads), 0, s, (const float*)o, o_head, (const float*)gate,
                                            ld_gate, (float*)out, heads, vdim, total), "sigmoid_gate");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(sigmoid_gate_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, (const __nv_bfloat16*)o, o_head,
                                            (const __nv_bfloat16*)gate, ld_gate, (__nv_bfloat16*)out, heads, vdim, total), "sigmoid_gate");
    else
        RMX_FAIL("sigmoid_gate: unknown dtype %d", dtype);
    return 0;
}
