// Attention over a cache of latents (see attention_latent.cu for the formulas) on tensor cores.
//
// The bfloat16 kernel on m16n8k16 tensor-core instructions.
//
// A CTA owns 64 rows, a row being one (token, head) pair; all rows of a CTA read the same
// latent tiles, which is what makes the shared latent pay: a tile of 64 cached positions is
// fetched once (asynchronous 16-byte copies, page by page, into double-buffered swizzled shared
// memory) and serves as the keys of S = Q' C^T and, read transposed, as the values of O += P C.
//   * prompt portions: 16 consecutive tokens of a request x 4 heads (`tokb` = 16); the four
//     16-row MMA tiles are the four heads;
//   * single-token requests: 1 token x 64 heads (`tokb` = 1), and the request's keys are cut into
//     chunks of `chunk` positions, one CTA (blockIdx.z) each, whose partial sums (float32, with
//     their maximum and denominator) a merge kernel adds up; with one chunk the CTA writes the
//     result itself.
// RT is the latent width rounded up to 64/128/256/512 (columns beyond the width are zeros in
// shared memory).  Up to RT = 256 a warp owns 16 rows and all columns of O (four warps); at
// RT = 512 two warps share a row tile (eight warps: registers hold 16 x 256 accumulators at
// most): each computes the scores of half of a tile's keys, they exchange row maxima, row sums
// and P (in the MMA's register layout) through shared memory at two barriers of their own, and
// each accumulates half of the output columns.  Softmax: online, float32,
// base 2; the sink enters as the starting maximum with denominator 1 (or in the merge).
#include "mma.cuh"

namespace somi {

constexpr int kLtRows = 64;
constexpr int kLtBN = 64;

// One tile of 64 cached positions.  A row (position) belongs to THREADS / 64 threads, which
// take its 16-byte pieces in turn: one look-up in the block table and one division a thread.
template <int RT, int THREADS>
__device__ __forceinline__ void load_latent_tile(unsigned char* dst,
                                                 const __nv_bfloat16* __restrict__ cache,
                                                 const int* __restrict__ bt, int kb, int k_lo,
                                                 int k_hi, int R, int page_size, int tid) {
    constexpr int CPR = RT / 8;
    constexpr int TPR = THREADS / kLtBN;                 // threads per row
    const int r = tid / TPR, sub = tid - r * TPR;
    const int j = kb + r;
    const bool row_ok = j >= k_lo && j < k_hi;
    size_t base = 0;
    if (row_ok) {
        const int page = bt[j / page_size];
        base = (static_cast<size_t>(page) * page_size + j % page_size) * R;
    }
#pragma unroll 4
    for (int ch = sub; ch < CPR; ch += TPR) {
        const bool ok = row_ok && ch * 8 < R;
        cp_async_16(smem_u32(dst + swizzled_offset<RT>(r, ch)), cache + (ok ? base + ch * 8 : 0),
                    ok ? 16 : 0);
    }
}

// The two warps of a row tile (warps mt and mt + 4) meet at a barrier of their own.
__device__ __forceinline__ void pair_barrier(int mt) {
    asm volatile("bar.sync %0, 64;\n" ::"r"(mt + 1) : "memory");
}
constexpr int kLtExchangeBytes = 4096 + 4 * 2 * 2 * 4 * 32 * 4;     // maxima, sums, P (12 KB)

template <int RT, int CSPLIT>
__global__ void __launch_bounds__(128 * CSPLIT)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, long long q_tok_stride,
                            long long q_head_stride, const __nv_bfloat16* __restrict__ cache,
                            const int* __restrict__ block_table, int bt_stride,
                            const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                            const int* __restrict__ tiles, int req_base, int row_base, int tokb,
                            int H, int R, int page_size, float scale_log2e, int window,
                            const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out,
                            long long o_tok_stride, long long o_head_stride, int chunk,
                            float* __restrict__ part_o, float* __restrict__ part_ml,
                            int max_splits) {
    constexpr int CPR = RT / 8;
    constexpr int TILE = kLtBN * RT * 2;
    constexpr int THREADS = 128 * CSPLIT;
    constexpr int OC = RT / 8 / CSPLIT;                 // 8-column output tiles per warp
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* Qs = smem_raw;                        // [64][RT]
    unsigned char* Cs = Qs + kLtRows * RT * 2;           // 2 x [64][RT]
    unsigned char* xch = Cs + 2 * TILE;                  // CSPLIT == 2: what warp pairs exchange
    pdl_launch_dependents();
    pdl_wait();

    int req, row0, rows;
    if (tiles) {
        const int tile = gridDim.x - 1 - blockIdx.x;     // later tiles see more keys: first
        req = tiles[3 * tile];
        row0 = tiles[3 * tile + 1];
        rows = tiles[3 * tile + 2];
    } else {
        req = req_base + blockIdx.x;
        row0 = row_base + blockIdx.x;
        rows = 1;
    }
    const int hb = kLtRows / tokb;                       // heads per CTA
    const int head0 = blockIdx.y * hb;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mt = warp & 3, cs = warp >> 2;
    const int q_pos0 = ctx_len[req] + (row0 - cu_q[req]);
    const int kv_end = q_pos0 + rows;
    const int kv_first = window > 0 ? max(0, q_pos0 - window + 1) : 0;
    const int kb_first = (kv_first / kLtBN) * kLtBN;
    // this CTA's share of the keys: chunk blockIdx.z, counted from the first key tile
    int k_lo = kv_first, k_hi = kv_end, kb0 = kb_first;
    if (chunk > 0) {
        kb0 = kb_first + blockIdx.z * chunk;
        k_lo = max(kv_first, kb0);
        k_hi = min(kv_end, kb0 + chunk);
    }
    const int* bt = block_table + static_cast<size_t>(req) * bt_stride;
    const int n_tiles = k_hi > kb0 ? (k_hi - kb0 + kLtBN - 1) / kLtBN : 0;

    for (int c = tid; c < kLtRows * CPR; c += THREADS) {
        const int r = c / CPR, ch = c - r * CPR;
        const int tok = r % tokb, head = head0 + r / tokb;
        const bool ok = tok < rows && head < H && ch * 8 < R;
        const __nv_bfloat16* src = q;
        if (ok) src = q + static_cast<size_t>(row0 + tok) * q_tok_stride +
                      static_cast<size_t>(head) * q_head_stride + ch * 8;
        cp_async_16(smem_u32(Qs + swizzled_offset<RT>(r, ch)), src, ok ? 16 : 0);
    }
    if (n_tiles > 0) load_latent_tile<RT, THREADS>(Cs, cache, bt, kb0, k_lo, k_hi, R, page_size, tid);
    cp_async_commit();

    float o[OC][4];
#pragma unroll
    for (int a = 0; a < OC; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) o[a][b] = 0.f;
    const int qr = mt * 16;
    const int row_lo = qr + (lane >> 2), row_hi = row_lo + 8;
    const int head_lo = head0 + row_lo / tokb, head_hi = head0 + row_hi / tokb;
    const int pos_lo = q_pos0 + row_lo % tokb, pos_hi = q_pos0 + row_hi % tokb;
    const bool ok_lo = row_lo % tokb < rows && head_lo < H, ok_hi = row_hi % tokb < rows && head_hi < H;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    if (sinks && chunk == 0) {
        // the sink: a key of score sinks[head] without a value, counted once
        if (ok_lo) { m_lo = sinks[head_lo] * 1.4426950408889634f; l_lo = 1.f; }
        if (ok_hi) { m_hi = sinks[head_hi] * 1.4426950408889634f; l_hi = 1.f; }
    }
    const bool warp_live = head0 + qr / tokb < H;        // any row of this warp's tile is a head

    for (int t = 0; t < n_tiles; ++t) {
        const int kb = kb0 + t * kLtBN;
        const int buf = t & 1;
        if (t + 1 < n_tiles)
            load_latent_tile<RT, THREADS>(Cs + (buf ^ 1) * TILE, cache, bt, kb + kLtBN, k_lo, k_hi, R,
                                          page_size, tid);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char* Ct = Cs + buf * TILE;
        if (warp_live) {
            // the 16-key groups whose scores this warp computes: all four, or (two warps a row
            // tile) its half of them; the other half comes from the partner through `xch`
            constexpr int NP = 4 / CSPLIT;
            const int np0 = cs * NP;
            float s[2 * NP][4];
#pragma unroll
            for (int a = 0; a < 2 * NP; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) s[a][b] = 0.f;
#pragma unroll 8
            for (int ks = 0; ks < RT / 16; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a, smem_u32(Qs + swizzled_offset<RT>(qr + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                                2 * ks + (lane >> 4))));
#pragma unroll
                for (int np = 0; np < NP; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, smem_u32(Ct + swizzled_offset<RT>((np0 + np) * 16 + (lane & 7) + (lane >> 4) * 8,
                                                                    2 * ks + ((lane >> 3) & 1))));
                    mma_bf16_16816(s[2 * np], a, b[0], b[1]);
                    mma_bf16_16816(s[2 * np + 1], a, b[2], b[3]);
                }
            }
            float t_lo = -INFINITY, t_hi = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2 * NP; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = kb + (2 * np0 + nt) * 8 + (lane & 3) * 2 + (e & 1);
                    const int pos = e < 2 ? pos_lo : pos_hi;
                    const bool ok = key <= pos && key >= k_lo && key < k_hi &&
                                    (window <= 0 || key > pos - window);
                    const float v = ok ? s[nt][e] * scale_log2e : -INFINITY;
                    s[nt][e] = v;
                    if (e < 2) t_lo = fmaxf(t_lo, v); else t_hi = fmaxf(t_hi, v);
                }
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 1));
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 2));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 1));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 2));
            if constexpr (CSPLIT == 2) {
                // the row maxima of the partner's keys
                float2* xmax = reinterpret_cast<float2*>(xch) + (mt * 2) * 32;
                xmax[cs * 32 + lane] = make_float2(t_lo, t_hi);
                pair_barrier(mt);
                const float2 other = xmax[(cs ^ 1) * 32 + lane];
                t_lo = fmaxf(t_lo, other.x);
                t_hi = fmaxf(t_hi, other.y);
            }
            const float n_lo = fmaxf(m_lo, t_lo), n_hi = fmaxf(m_hi, t_hi);
            const float b_lo = n_lo == -INFINITY ? 0.f : n_lo, b_hi = n_hi == -INFINITY ? 0.f : n_hi;
            const float a_lo = exp2f(m_lo - b_lo), a_hi = exp2f(m_hi - b_hi);
            m_lo = n_lo;
            m_hi = n_hi;
            float r_lo = 0.f, r_hi = 0.f;
            uint32_t own[NP][4];
#pragma unroll
            for (int nt = 0; nt < 2 * NP; ++nt) {
                const uint32_t lo = pack_bf16(exp2f(s[nt][0] - b_lo), exp2f(s[nt][1] - b_lo));
                const uint32_t hi = pack_bf16(exp2f(s[nt][2] - b_hi), exp2f(s[nt][3] - b_hi));
                const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&lo);
                const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&hi);
                r_lo += __low2float(lo2) + __high2float(lo2);
                r_hi += __low2float(hi2) + __high2float(hi2);
                own[nt >> 1][(nt & 1) * 2] = lo;
                own[nt >> 1][(nt & 1) * 2 + 1] = hi;
            }
            r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 1);
            r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 2);
            r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 1);
            r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 2);
            uint32_t pa[4][4];
            if constexpr (CSPLIT == 1) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
#pragma unroll
                    for (int e = 0; e < 4; ++e) pa[k][e] = own[k % NP][e];
            }
            if constexpr (CSPLIT == 2) {
                // P of this warp's keys, in the MMA's own register layout (both warps of a row
                // tile hold the same rows in the same lanes), and its row sums
                float2* xsum = reinterpret_cast<float2*>(xch + 2048) + (mt * 2) * 32;
                uint32_t* xp = reinterpret_cast<uint32_t*>(xch + 4096) + (mt * 2) * (NP * 4 * 32);
                xsum[cs * 32 + lane] = make_float2(r_lo, r_hi);
#pragma unroll
                for (int k = 0; k < NP; ++k)
#pragma unroll
                    for (int e = 0; e < 4; ++e) xp[cs * (NP * 4 * 32) + (k * 4 + e) * 32 + lane] = own[k][e];
                pair_barrier(mt);
                const float2 other = xsum[(cs ^ 1) * 32 + lane];
                // the same order of addition in both warps: first half's keys, then second half's
                r_lo = cs == 0 ? r_lo + other.x : other.x + r_lo;
                r_hi = cs == 0 ? r_hi + other.y : other.y + r_hi;
#pragma unroll
                for (int k = 0; k < NP; ++k)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t oth = xp[(cs ^ 1) * (NP * 4 * 32) + (k * 4 + e) * 32 + lane];
                        pa[k % 4][e] = cs == 0 ? own[k][e] : oth;                  // keys 0..31
                        pa[(NP + k) % 4][e] = cs == 0 ? oth : own[k][e];           // keys 32..63
                    }
            }
            l_lo = l_lo * a_lo + r_lo;
            l_hi = l_hi * a_hi + r_hi;
#pragma unroll
            for (int nt = 0; nt < OC; ++nt) {
                o[nt][0] *= a_lo; o[nt][1] *= a_lo;
                o[nt][2] *= a_hi; o[nt][3] *= a_hi;
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                for (int dc = 0; dc < OC / 2; ++dc) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, smem_u32(Ct + swizzled_offset<RT>(
                                             kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                             2 * (cs * (OC / 2) + dc) + (lane >> 4))));
                    mma_bf16_16816(o[2 * dc], pa[kk], b[0], b[1]);
                    mma_bf16_16816(o[2 * dc + 1], pa[kk], b[2], b[3]);
                }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    if (chunk == 0) {
        const float i_lo = l_lo > 0.f ? 1.0f / l_lo : 0.f, i_hi = l_hi > 0.f ? 1.0f / l_hi : 0.f;
#pragma unroll
        for (int nt = 0; nt < OC; ++nt) {
            const int d = (cs * OC + nt) * 8 + (lane & 3) * 2;
            if (d >= R) continue;
            if (ok_lo)
                *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(row0 + row_lo % tokb) * o_tok_stride +
                                             static_cast<size_t>(head_lo) * o_head_stride + d) =
                    pack_bf16(o[nt][0] * i_lo, o[nt][1] * i_lo);
            if (ok_hi)
                *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(row0 + row_hi % tokb) * o_tok_stride +
                                             static_cast<size_t>(head_hi) * o_head_stride + d) =
                    pack_bf16(o[nt][2] * i_hi, o[nt][3] * i_hi);
        }
        return;
    }
    // partial sums of this chunk (tokb == 1: the row is the head), unnormalised
    const int i = blockIdx.x;
    const size_t p_lo = (static_cast<size_t>(i) * H + head_lo) * max_splits + blockIdx.z;
    const size_t p_hi = (static_cast<size_t>(i) * H + head_hi) * max_splits + blockIdx.z;
#pragma unroll
    for (int nt = 0; nt < OC; ++nt) {
        const int d = (cs * OC + nt) * 8 + (lane & 3) * 2;
        if (d >= R) continue;
        if (ok_lo) *reinterpret_cast<float2*>(part_o + p_lo * R + d) = make_float2(o[nt][0], o[nt][1]);
        if (ok_hi) *reinterpret_cast<float2*>(part_o + p_hi * R + d) = make_float2(o[nt][2], o[nt][3]);
    }
    if (cs == 0 && (lane & 3) == 0) {
        if (ok_lo) *reinterpret_cast<float2*>(part_ml + 2 * p_lo) = make_float2(m_lo, l_lo);
        if (ok_hi) *reinterpret_cast<float2*>(part_ml + 2 * p_hi) = make_float2(m_hi, l_hi);
    }
}

// out[h][row] = sum_s 2^(m_s - M) o_s / (sum_s 2^(m_s - M) l_s + 2^(sink_h log2 e - M)) over the
// chunks that held keys; M is the maximum over the chunks and the sink.
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    int max_splits, int n_splits, int H, int R,
                                    const float* __restrict__ sinks, int row_base,
                                    __nv_bfloat16* __restrict__ out, long long o_tok_stride,
                                    long long o_head_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x, head = blockIdx.y;
    const size_t base = (static_cast<size_t>(i) * H + head) * max_splits;
    const float sink = sinks ? sinks[head] * 1.4426950408889634f : -INFINITY;
    float M = sink;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[2 * (base + s)]);
    float L = sinks ? exp2f(sink - M) : 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float m = part_ml[2 * (base + s)];
        if (m != -INFINITY) L += exp2f(m - M) * part_ml[2 * (base + s) + 1];
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int d = threadIdx.x; d < R; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float m = part_ml[2 * (base + s)];
            if (m != -INFINITY) acc += exp2f(m - M) * part_o[(base + s) * R + d];
        }
        out[static_cast<size_t>(row_base + i) * o_tok_stride + static_cast<size_t>(head) * o_head_stride + d] =
            __float2bfloat16_rn(acc * inv);
    }
}

template <int RT, int CSPLIT>
int launch_latent_mma(dim3 grid, cudaStream_t stream, const void* q, long long qts, long long qhs,
                      const void* cache, const int* block_table, int bt_stride, const int* cu_q,
                      const int* ctx_len, const int* tiles, int req_base, int row_base, int tokb,
                      int H, int R, int page_size, float scale, int window, const float* sinks,
                      void* out, long long ots, long long ohs, int chunk, float* part_o,
                      float* part_ml, int max_splits) {
    const size_t smem = static_cast<size_t>(kLtRows + 2 * kLtBN) * RT * 2 +
                        (CSPLIT == 2 ? kLtExchangeBytes : 0);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(latent_attention_mma_kernel<RT, CSPLIT>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_pdl(latent_attention_mma_kernel<RT, CSPLIT>, grid, dim3(128 * CSPLIT), smem, stream,
                      static_cast<const __nv_bfloat16*>(q), qts, qhs,
                      static_cast<const __nv_bfloat16*>(cache), block_table, bt_stride, cu_q, ctx_len,
                      tiles, req_base, row_base, tokb, H, R, page_size,
                      scale * 1.4426950408889634f, window, sinks, static_cast<__nv_bfloat16*>(out),
                      ots, ohs, chunk, part_o, part_ml, max_splits);
}

}  // namespace somi

using namespace somi;

SOMI_API int somi_latent_attention_mma_q_tile() { return 16; }
SOMI_API int somi_latent_attention_mma_supported(int heads, int R) {
    return heads >= 1 && heads <= 65535 * 4 && R >= 8 && R <= 512 && R % 8 == 0;
}

// bfloat16.  `tiles`: int32 [n_tiles, 3] = (request, first row, rows <= 16) over the multi-token
// requests; the n_decode single-token requests follow them (request n_prefill_req + i, row
// n_prefill_tok + i).  `max_kv_len`: the longest request's keys after this step.  `scratch`:
// float32, at least n_decode * heads * splits * (R + 2) elements where splits =
// somi_latent_attention_mma_splits(max_kv_len, window, n_decode, heads) > 1.
// Keys per chunk of a single-token request: a multiple of the key tile, as small as keeps the
// step's CTAs (requests x head groups x chunks) within two per SM.  A short chunk means a short
// chain of tiles per CTA, which is what a decode step waits for.
static int latent_chunk(int max_kv_len, int window, int n_decode, int heads) {
    const int span = window > 0 ? min(window + kLtBN, max_kv_len) : max_kv_len;
    const int tiles = max(1, (span + kLtBN - 1) / kLtBN);
    const int groups = max(1, n_decode) * ((heads + kLtRows - 1) / kLtRows);
    const int splits = max(1, min(tiles, (2 * 148) / groups));
    return ((tiles + splits - 1) / splits) * kLtBN;
}

SOMI_API int somi_latent_attention_mma_splits(int max_kv_len, int window, int n_decode, int heads) {
    const int span = window > 0 ? min(window + kLtBN, max_kv_len) : max_kv_len;
    const int chunk = latent_chunk(max_kv_len, window, n_decode, heads);
    return max(1, (span + chunk - 1) / chunk);
}

SOMI_API int somi_latent_attention_mma(
    const void* q, long long q_tok_stride, long long q_head_stride, const void* cache,
    const int* block_table, int bt_stride, const int* cu_q, const int* ctx_len, const int* tiles,
    int n_tiles, int n_prefill_req, int n_prefill_tok, int n_decode, int max_kv_len, int heads,
    int R, int page_size, float scale, int window, const float* sinks, void* out,
    long long o_tok_stride, long long o_head_stride, float* scratch, cudaStream_t stream) {
    if (n_tiles + n_decode <= 0) return 0;
    if (!somi_latent_attention_mma_supported(heads, R) || page_size <= 0 ||
        (q_tok_stride | q_head_stride | o_tok_stride | o_head_stride) % 8 ||
        (reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache)) % 16)
        return SOMI_ERR_UNSUPPORTED;
    const int splits = n_decode > 0 ? somi_latent_attention_mma_splits(max_kv_len, window, n_decode, heads) : 1;
    const int chunk = latent_chunk(max_kv_len, window, n_decode, heads);
    if (splits > 65535) return SOMI_ERR_UNSUPPORTED;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + static_cast<size_t>(n_decode) * heads * splits * R : nullptr;
    if (splits > 1 && !scratch) return SOMI_ERR_UNSUPPORTED;
    int rc = 0;
#define SOMI_LATT_MMA(RT, CS)                                                                   \
    do {                                                                                        \
        if (n_tiles > 0)                                                                        \
            rc = launch_latent_mma<RT, CS>(dim3(n_tiles, (heads + 3) / 4), stream, q,           \
                q_tok_stride, q_head_stride, cache, block_table, bt_stride, cu_q, ctx_len,      \
                tiles, 0, 0, 16, heads, R, page_size, scale, window, sinks, out, o_tok_stride,  \
                o_head_stride, 0, nullptr, nullptr, 1);                                         \
        if (rc == 0 && n_decode > 0)                                                            \
            rc = launch_latent_mma<RT, CS>(dim3(n_decode, (heads + 63) / 64, splits), stream,   \
                q, q_tok_stride, q_head_stride, cache, block_table, bt_stride, cu_q, ctx_len,   \
                nullptr, n_prefill_req, n_prefill_tok, 1, heads, R, page_size, scale, window,   \
                sinks, out, o_tok_stride, o_head_stride, splits > 1 ? chunk : 0, part_o, part_ml,\
                splits);                                                                        \
    } while (0)
    if (R <= 64) SOMI_LATT_MMA(64, 1);
    else if (R <= 128) SOMI_LATT_MMA(128, 1);
    else if (R <= 256) SOMI_LATT_MMA(256, 1);
    else SOMI_LATT_MMA(512, 2);
#undef SOMI_LATT_MMA
    if (rc != 0) return rc;
    if (n_decode > 0 && splits > 1)
        launch_pdl(latent_merge_kernel, dim3(n_decode, heads), dim3(min(256, ((R + 31) / 32) * 32)), 0,
                   stream, part_o, part_ml, splits, splits, heads, R, sinks, n_prefill_tok,
                   static_cast<__nv_bfloat16*>(out), o_tok_stride, o_head_stride);
    return launch_status();
}
