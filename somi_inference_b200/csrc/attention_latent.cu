// Attention over a cache of latents: every head reads the same cached vector per position, as
// key and as value (multi-query attention whose keys are its values), with a sliding window and
// an optional sink per head.  The caller has folded the key expansion into the queries
// (q'_h = W_uk,h^T q_h, so that q_h . k_h = q'_h . c) and applies the value expansion to the
// result (W_uv,h sum_j p_j c_j), which is why only the latent c is cached.
//
//   s_ij = scale * q'_i . c_j          for max(0, i - window + 1) <= j <= i   (window 0: all j <= i)
//   p_ij = exp(s_ij - m_i) / (sum_j exp(s_ij - m_i) + exp(sink_h - m_i)),  m_i = max(sink_h, max_j s_ij)
//   o_i  = sum_j p_ij c_j
// The sink adds to the denominator only: a key whose score is sink_h and whose value is zero.
//
// This file holds the kernel on the CUDA cores for any dtype and any latent width up to 512 (the
// float32 path's kernel, and the bfloat16 path's for widths the tensor-core kernel of
// attention_latent_mma.cu refuses).
// Key tiles are aligned to multiples of kBN from position 0 and the softmax is online in
// float32, so a row's arithmetic does not depend on how its request was cut into steps.
//
// One CTA = one q tile (<= kBM consecutive tokens of one request) x one head.  Tiles [0, n_tiles)
// come from the tile list (request, first row, rows); CTAs beyond them are the single-token
// requests: request n_prefill_req + i, row n_prefill_tok + i.
#include "common.cuh"

namespace somi {

constexpr int kLBM = 16;
constexpr int kLBN = 32;
constexpr int kLThreads = 128;
constexpr int kLMaxR = 512;
constexpr int kLAcc = kLBM * kLMaxR / kLThreads;     // 64

template <typename T>
__global__ void __launch_bounds__(kLThreads)
latent_attention_generic_kernel(const T* __restrict__ q, long long q_tok_stride,
                                long long q_head_stride, const T* __restrict__ cache,
                                const int* __restrict__ block_table, int bt_stride,
                                const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                                const int* __restrict__ tiles, int n_tiles, int n_prefill_req,
                                int n_prefill_tok, int R, int page_size, float scale, int window,
                                const float* __restrict__ sinks, T* __restrict__ out,
                                long long o_tok_stride, long long o_head_stride) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    float* Qs = smem;                           // [kLBM][R]
    float* Cs = Qs + kLBM * R;                  // [kLBN][R + 1]
    float* Ss = Cs + kLBN * (R + 1);            // [kLBM][kLBN + 1]
    float* m_s = Ss + kLBM * (kLBN + 1);        // [kLBM]
    float* l_s = m_s + kLBM;
    float* a_s = l_s + kLBM;

    int req, row0, rows;
    if (static_cast<int>(blockIdx.x) < n_tiles) {
        req = tiles[3 * blockIdx.x];
        row0 = tiles[3 * blockIdx.x + 1];
        rows = tiles[3 * blockIdx.x + 2];
    } else {
        const int i = blockIdx.x - n_tiles;
        req = n_prefill_req + i;
        row0 = n_prefill_tok + i;
        rows = 1;
    }
    const int head = blockIdx.y;
    const int tid = threadIdx.x;
    const int q_pos0 = ctx_len[req] + (row0 - cu_q[req]);
    const int kv_end = q_pos0 + rows;                                    // exclusive
    const int kv_first = window > 0 ? max(0, q_pos0 - window + 1) : 0;    // first key any row reads
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;
    const int Rp = R + 1;

    for (int idx = tid; idx < kLBM * R; idx += kLThreads) {
        const int m = idx / R, d = idx - m * R;
        Qs[idx] = m < rows ? to_float(q[static_cast<size_t>(row0 + m) * q_tok_stride +
                                        static_cast<size_t>(head) * q_head_stride + d]) * scale
                           : 0.f;
    }
    if (tid < kLBM) {
        // the sink: a key with score sinks[head] and no value, counted once
        m_s[tid] = sinks ? sinks[head] : -INFINITY;
        l_s[tid] = sinks ? 1.f : 0.f;
    }
    float acc[kLAcc];
#pragma unroll
    for (int i = 0; i < kLAcc; ++i) acc[i] = 0.f;
    __syncthreads();

    for (int kb = (kv_first / kLBN) * kLBN; kb < kv_end; kb += kLBN) {
        for (int idx = tid; idx < kLBN * R; idx += kLThreads) {
            const int n = idx / R, d = idx - n * R;
            const int j = kb + n;
            float c = 0.f;
            if (j >= kv_first && j < kv_end) {
                const int page = bt[j / page_size];
                c = to_float(cache[(static_cast<size_t>(page) * page_size + j % page_size) * R + d]);
            }
            Cs[n * Rp + d] = c;
        }
        __syncthreads();
        for (int idx = tid; idx < kLBM * kLBN; idx += kLThreads) {
            const int m = idx / kLBN, n = idx - m * kLBN;
            const int j = kb + n, qp = q_pos0 + m;
            float s = -INFINITY;
            if (m < rows && j <= qp && j >= kv_first && (window <= 0 || j > qp - window)) {
                s = 0.f;
                const float* qr = Qs + m * R;
                const float* cr = Cs + n * Rp;
                for (int d = 0; d < R; ++d) s = fmaf(qr[d], cr[d], s);
            }
            Ss[m * (kLBN + 1) + n] = s;
        }
        __syncthreads();
        {   // online softmax: one warp per row, one key per lane (kLBN == 32)
            const int warp = tid >> 5, lane = tid & 31;
            for (int m = warp; m < kLBM; m += kLThreads / 32) {
                const float s = Ss[m * (kLBN + 1) + lane];
                const float m_old = m_s[m];
                const float m_new = fmaxf(m_old, warp_max(s));
                float p = 0.f, alpha = 1.f;
                if (m_new != -INFINITY) {
                    alpha = expf(m_old - m_new);
                    p = expf(s - m_new);
                }
                const float psum = warp_sum(p);
                Ss[m * (kLBN + 1) + lane] = p;
                if (lane == 0) {
                    m_s[m] = m_new;
                    l_s[m] = l_s[m] * alpha + psum;
                    a_s[m] = alpha;
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kLAcc; ++i) {
            const int idx = tid + i * kLThreads;
            if (idx < kLBM * R) {
                const int m = idx / R, d = idx - m * R;
                float o = acc[i] * a_s[m];
                const float* p = Ss + m * (kLBN + 1);
#pragma unroll 4
                for (int n = 0; n < kLBN; ++n) o = fmaf(p[n], Cs[n * Rp + d], o);
                acc[i] = o;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < kLAcc; ++i) {
        const int idx = tid + i * kLThreads;
        if (idx < kLBM * R) {
            const int m = idx / R, d = idx - m * R;
            if (m < rows)
                out[static_cast<size_t>(row0 + m) * o_tok_stride +
                    static_cast<size_t>(head) * o_head_stride + d] = from_float<T>(acc[i] / l_s[m]);
        }
    }
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_latent_attention_generic_q_tile() { return kLBM; }

// q, out: element (token t, head h, d) at t * tok_stride + h * head_stride + d.
// cache: [pages, page_size, R].  sinks: float32 [heads] or null.
SOMI_API int somi_latent_attention_generic(
    const void* q, int dtype, long long q_tok_stride, long long q_head_stride, const void* cache,
    const int* block_table, int bt_stride, const int* cu_q, const int* ctx_len, const int* tiles,
    int n_tiles, int n_prefill_req, int n_prefill_tok, int n_decode, int heads, int R,
    int page_size, float scale, int window, const float* sinks, void* out, long long o_tok_stride,
    long long o_head_stride, cudaStream_t stream) {
    if (n_tiles + n_decode <= 0) return 0;
    if (R <= 0 || R > kLMaxR || heads <= 0 || heads > 65535 || page_size <= 0)
        return SOMI_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * (static_cast<size_t>(kLBM) * R + kLBN * (R + 1) +
                                         kLBM * (kLBN + 1) + 3 * kLBM);
    dim3 grid(n_tiles + n_decode, heads);
#define SOMI_LAUNCH_LATT(T)                                                                     \
    do {                                                                                        \
        if (smem > 48 * 1024)                                                                   \
            cudaFuncSetAttribute(latent_attention_generic_kernel<T>,                            \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        launch_pdl(latent_attention_generic_kernel<T>, dim3(grid), dim3(kLThreads), smem,       \
            stream, static_cast<const T*>(q), q_tok_stride, q_head_stride,                      \
            static_cast<const T*>(cache), block_table, bt_stride, cu_q, ctx_len, tiles,         \
            n_tiles, n_prefill_req, n_prefill_tok, R, page_size, scale, window, sinks,          \
            static_cast<T*>(out), o_tok_stride, o_head_stride);                                 \
    } while (0)
    if (dtype == SOMI_F32) SOMI_LAUNCH_LATT(float);
    else SOMI_LAUNCH_LATT(__nv_bfloat16);
#undef SOMI_LAUNCH_LATT
    return launch_status();
}
