// Pieces of attention through a cached latent: the two RMS norms after the down projections (the key/value
// latent goes straight into its page), and the per-head output gate.
//
// A mixer of this kind projects its input to a query latent and a key/value latent, both much narrower than
// heads * head size, norms each, and keeps only the key/value latent per token; keys and values are products
// of that latent with per-head weights.  Norms are formed in float whatever the activations' type.
#include "common.cuh"

namespace {
constexpr int THREADS = 128;

// One block per token.  row = proj[t] holds [query latent (q_rank) | key/value latent (kv_rank) | ...].
//   cq[t]   = row[0 : q_rank]            / sqrt(mean(.^2) + eps) * wq
//   page[t] = row[q_rank : q_rank + kv]  / sqrt(mean(.^2) + eps) * wkv     (kv_rank 0: the layer reads another's latents)
// The order of every sum depends on the sizes only.
template <typename T>
__global__ void __launch_bounds__(THREADS) latent_norms_kernel(
    const T* __restrict__ proj, int ld, int q_rank, int kv_rank, const float* __restrict__ wq,
    const float* __restrict__ wkv, float eps, T* __restrict__ cq, T* __restrict__ pool,
    const int* __restrict__ positions, const int* __restrict__ seq_index, const int* __restrict__ block_table,
    int table_stride, int page_size, int* __restrict__ status) {
    __shared__ float scratch[32];
    allow_dependents();
    wait_for_prior_kernels();
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * ld;
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += THREADS) {
        const float v = to_float(row[i]);
        ss += v * v;
    }
    const float inv_q = rsqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += THREADS)
        cq[(size_t)t * q_rank + i] = from_float<T>(to_float(row[i]) * inv_q * wq[i]);
    if (kv_rank == 0 || pool == nullptr) return;
    const T* kv = row + q_rank;
    ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += THREADS) {
        const float v = to_float(kv[i]);
        ss += v * v;
    }
    const float inv_kv = rsqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
    const int pos = positions[t];
    const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
    if (page < 0) {
        if (threadIdx.x == 0) atomicExch(status, 1);  // a latent was to be written to a position without a page
        return;
    }
    T* dst = pool + ((size_t)page * page_size + pos % page_size) * kv_rank;
    for (int i = threadIdx.x; i < kv_rank; i += THREADS) dst[i] = from_float<T>(to_float(kv[i]) * inv_kv * wkv[i]);
}

// o[t, h, :] *= sigmoid(gate[t, h]), gate rows ld_gate apart (columns of the down projection's output).
template <typename T>
__global__ void gate_heads_kernel(T* __restrict__ o, const T* __restrict__ gate, int ld_gate, int heads, int vdim,
                                  size_t total) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t per_row = (size_t)heads * vdim;
    const size_t t = idx / per_row;
    const int h = (int)((idx - t * per_row) / vdim);
    const float g = to_float(gate[t * ld_gate + h]);
    o[idx] = from_float<T>(to_float(o[idx]) / (1.f + expf(-g)));
}

// bfloat16, eight numbers a thread (16-byte accesses); vdim is a multiple of 8.
__global__ void gate_heads8_kernel(__nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ gate, int ld_gate, int heads,
                                   int vdim, size_t total8) {
    allow_dependents();
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total8) return;
    const size_t per_row = (size_t)heads * vdim / 8;
    const size_t t = idx / per_row;
    const int h = (int)((idx - t * per_row) * 8 / vdim);
    const float g = __bfloat162float(gate[t * ld_gate + h]);
    const float f = 1.f / (1.f + expf(-g));
    uint4 raw = *reinterpret_cast<const uint4*>(o + idx * 8);
    uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[j]));
        __nv_bfloat162 r = __floats2bfloat162_rn(v.x * f, v.y * f);
        words[j] = *reinterpret_cast<uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(o + idx * 8) = make_uint4(words[0], words[1], words[2], words[3]);
}
}  // namespace

RMX_API int rmx_latent_norms(const void* proj, int ld, int q_rank, int kv_rank, const float* wq, const float* wkv,
                             float eps, void* cq, void* pool, const int* positions, const int* seq_index,
                             const int* block_table, int table_stride, int page_size, int n_tokens, int* status,
                             int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && q_rank > 0 && kv_rank >= 0 && ld >= q_rank + kv_rank, "latent_norms: bad sizes");
    RMX_REQUIRE(proj && wq && cq, "latent_norms: a null pointer");
    RMX_REQUIRE(kv_rank == 0 || pool == nullptr || (wkv && positions && seq_index && block_table && table_stride > 0 && page_size > 0 && status),
                "latent_norms: writing latents needs their norm's weight, positions, the block table and a status word");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(latent_norms_kernel<float>, dim3(n_tokens), dim3(THREADS), 0, s, (const float*)proj, ld, q_rank,
                                            kv_rank, wq, wkv, eps, (float*)cq, (float*)pool, positions, seq_index, block_table,
                                            table_stride, page_size, status), "latent_norms");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(latent_norms_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(THREADS), 0, s,
                                            (const __nv_bfloat16*)proj, ld, q_rank, kv_rank, wq, wkv, eps, (__nv_bfloat16*)cq,
                                            (__nv_bfloat16*)pool, positions, seq_index, block_table, table_stride, page_size, status),
                           "latent_norms");
    else
        RMX_FAIL("latent_norms: unknown dtype %d", dtype);
    return 0;
}

RMX_API int rmx_gate_heads(void* o, const void* gate, int ld_gate, int n_tokens, int heads, int vdim, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && heads > 0 && vdim > 0 && ld_gate >= heads && o && gate, "gate_heads: bad sizes or a null pointer");
    const size_t total = (size_t)n_tokens * heads * vdim;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(gate_heads_kernel<float>, dim3(blocks), dim3(threads), 0, s, (float*)o, (const float*)gate,
                                            ld_gate, heads, vdim, total), "gate_heads");
    else if (dtype == RMX_BF16 && (vdim & 7) == 0 && ((uintptr_t)o & 15) == 0)
        RMX_CHECK_LAUNCHED(launch_dependent(gate_heads8_kernel, dim3((unsigned)((total / 8 + threads - 1) / threads)), dim3(threads), 0, s,
                                            (__nv_bfloat16*)o, (const __nv_bfloat16*)gate, ld_gate, heads, vdim, total / 8), "gate_heads");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(gate_heads_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (__nv_bfloat16*)o,
                                            (const __nv_bfloat16*)gate, ld_gate, heads, vdim, total), "gate_heads");
    else
        RMX_FAIL("gate_heads: unknown dtype %d", dtype);
    return 0;
}
