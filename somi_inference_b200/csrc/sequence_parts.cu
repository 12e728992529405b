// Kernels of layer parts that work along the sequence or around a residual branch, beside the
// ones of layer_parts.cu:
//   * token embedding times a constant -> float32 residual stream
//   * residual += rmsnorm(branch) * weight_b, then rmsnorm(residual) * weight ("sandwich" norms)
//   * short causal convolution over a range of columns of a wider product, with bias,
//     activation and a per-request state of the last inputs
//   * rotation of neighbouring pairs of q and k, unit root mean square per head, cache write
//     (keys and values of different widths)
//   * sigmoid gate on a mixer's output, soft cap on logits
//   * the state-space recurrence of a Mamba-2 mixer and its gated group norm
// Norms, angles, gates, decays and the recurrent state are float32; inputs and outputs are float32
// or bfloat16.
#include "common.cuh"
#include "vec4.cuh"

namespace somi {

// ---------------------------------------------------------------- scaled embedding
// out[t, :] = float(table[ids[t], :]) * scale
template <typename T>
__global__ void embed_scaled_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                    float scale, float* __restrict__ out, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = table + static_cast<size_t>(ids[t]) * H;
    float* o = out + static_cast<size_t>(t) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]) * scale;
}

// ------------------------------------------------ normed residual sum + RMS norm
// d = sum_s delta[s][row] (partial sums `split_stride` apart, added in order);
// r = residual[row] + d / sqrt(mean(d^2) + eps_b) * weight_b   (no delta: r = residual[row]);
// if write_back: residual[row] = r;  if out: out[b] = r / sqrt(mean(r^2) + eps) * weight,
// row = rows ? rows[b] : b.  The row lives in shared memory (H floats) between the passes.
template <typename TD, typename TO>
__global__ void add_normed_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                          int splits, long long split_stride,
                                          const void* __restrict__ weight_b, int wb_dtype, float eps_b,
                                          const void* __restrict__ weight, int w_dtype, float eps,
                                          TO* __restrict__ out, const int* __restrict__ rows, int H,
                                          int write_back, int vec4) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int row = rows ? rows[b] : b;
    float* res = residual + static_cast<size_t>(row) * H;
    float ss = 0.f;
    if (vec4) {
        // four columns a thread: with a thread per four columns (the launcher's choice for the few
        // rows of a decode step) every load of the row and of its partial sums is in flight at once
        if (delta != nullptr) {
            const TD* d0 = delta + static_cast<size_t>(row) * H;
            for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
                F4 d = load4(d0 + i);
#pragma unroll 4
                for (int s = 1; s < splits; ++s) {
                    const F4 e = load4(d0 + static_cast<size_t>(s) * split_stride + i);
#pragma unroll
                    for (int c = 0; c < 4; ++c) d.v[c] += e.v[c];
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) ss = fmaf(d.v[c], d.v[c], ss);
                store4(row_buf + i, d);
            }
            ss = block_sum(ss, scratch);
            const float rd = 1.0f / sqrtf(ss / static_cast<float>(H) + eps_b);
            ss = 0.f;
            for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
                const F4 d = load4(row_buf + i), wb = load4_any(weight_b, wb_dtype, i);
                F4 r = load4(res + i);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    r.v[c] += d.v[c] * rd * wb.v[c];
                    ss = fmaf(r.v[c], r.v[c], ss);
                }
                store4(row_buf + i, r);
                if (write_back) store4(res + i, r);
            }
        } else {
            for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
                const F4 r = load4(res + i);
#pragma unroll
                for (int c = 0; c < 4; ++c) ss = fmaf(r.v[c], r.v[c], ss);
                store4(row_buf + i, r);
            }
        }
        if (out == nullptr) return;
        ss = block_sum(ss, scratch);
        const float rr = 1.0f / sqrtf(ss / static_cast<float>(H) + eps);
        TO* o = out + static_cast<size_t>(b) * H;
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const F4 w = load4_any(weight, w_dtype, i);
            F4 r = load4(row_buf + i);
#pragma unroll
            for (int c = 0; c < 4; ++c) r.v[c] = r.v[c] * rr * w.v[c];
            store4(o + i, r);
        }
        return;
    }
    if (delta != nullptr) {
        const TD* d0 = delta + static_cast<size_t>(row) * H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float d = to_float(d0[i]);
            for (int s = 1; s < splits; ++s) d += to_float(d0[static_cast<size_t>(s) * split_stride + i]);
            row_buf[i] = d;
            ss = fmaf(d, d, ss);
        }
        ss = block_sum(ss, scratch);
        const float rd = 1.0f / sqrtf(ss / static_cast<float>(H) + eps_b);
        ss = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float r = res[i] + row_buf[i] * rd * load_as_float(weight_b, wb_dtype, i);
            row_buf[i] = r;
            if (write_back) res[i] = r;
            ss = fmaf(r, r, ss);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float r = res[i];
            row_buf[i] = r;
            ss = fmaf(r, r, ss);
        }
    }
    if (out == nullptr) return;
    ss = block_sum(ss, scratch);
    const float rr = 1.0f / sqrtf(ss / static_cast<float>(H) + eps);
    TO* o = out + static_cast<size_t>(b) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_float<TO>(row_buf[i] * rr * load_as_float(weight, w_dtype, i));
}

// ------------------------------------------------- short causal convolution, general form
// u: rows `in_stride` elements apart, C channels from the pointer on.
// out[t, c] = act(bias[c] + sum_{d=0}^{taps-1} w[taps-1-d, c] * u_(t-d)[c]) (+ u_t[c] if add_input),
// u_(t-d) being the row d places back in the same request: a row of this step or, before the
// step's first row, the request's state (its last taps-1 inputs, oldest first; zero before the
// sequence's start).  act 0: none, 1: silu.  The state is only read here.
template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ u, long long in_stride,
                                   const float* __restrict__ w, const float* __restrict__ bias,
                                   const T* __restrict__ state, const int* __restrict__ cu_q,
                                   const int* __restrict__ token_request,
                                   const int* __restrict__ state_slot, T* __restrict__ out,
                                   long long out_stride, int C, int taps, int act, int add_input,
                                   int n_tokens, int vec4) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x * blockDim.y + threadIdx.y;
    if (t >= n_tokens) return;
    const int req = token_request[t];
    const int local = t - cu_q[req];
    const T* st = state + static_cast<size_t>(state_slot[req]) * (taps - 1) * C;
    if (vec4) {
        for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < C; c += gridDim.y * blockDim.x * 4) {
            const F4 own = load4(u + static_cast<size_t>(t) * in_stride + c);
            F4 acc = F4{{0.f, 0.f, 0.f, 0.f}};
            for (int d = taps - 1; d >= 0; --d) {      // oldest input first
                const F4 v = d == 0 ? own
                             : (local - d >= 0 ? load4(u + static_cast<size_t>(t - d) * in_stride + c)
                                               : load4(st + static_cast<size_t>(taps - 1 + local - d) * C + c));
                const F4 ww = load4(w + static_cast<size_t>(taps - 1 - d) * C + c);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc.v[e] = fmaf(ww.v[e], v.v[e], acc.v[e]);
            }
            if (bias != nullptr) {
                const F4 bb = load4(bias + c);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc.v[e] += bb.v[e];
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (act == 1) acc.v[e] = acc.v[e] / (1.0f + expf(-acc.v[e]));
                if (add_input) acc.v[e] += own.v[e];
            }
            store4(out + static_cast<size_t>(t) * out_stride + c, acc);
        }
        return;
    }
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const float own = to_float(u[static_cast<size_t>(t) * in_stride + c]);
        float acc = 0.f;
        for (int d = taps - 1; d >= 0; --d) {          // oldest input first
            float v;
            if (d == 0) v = own;
            else if (local - d >= 0) v = to_float(u[static_cast<size_t>(t - d) * in_stride + c]);
            else v = to_float(st[static_cast<size_t>(taps - 1 + local - d) * C + c]);
            acc = fmaf(w[static_cast<size_t>(taps - 1 - d) * C + c], v, acc);
        }
        if (bias != nullptr) acc += bias[c];
        if (act == 1) acc = acc / (1.0f + expf(-acc));
        if (add_input) acc += own;
        out[static_cast<size_t>(t) * out_stride + c] = from_float<T>(acc);
    }
}

// New state of request r: its last taps-1 inputs after this step's rows, oldest first.  A thread
// owns one channel of one request and reads what it needs of the old state before it writes.
constexpr int kConvMaxTaps = 32;
template <typename T>
__global__ void causal_conv_state_kernel(const T* __restrict__ u, long long in_stride,
                                         T* __restrict__ state, const int* __restrict__ cu_q,
                                         const int* __restrict__ state_slot, int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int req = blockIdx.x;
    const int first = cu_q[req], q = cu_q[req + 1] - first;
    const int keep = taps - 1;
    T* st = state + static_cast<size_t>(state_slot[req]) * keep * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        T v[kConvMaxTaps];
        for (int s = 0; s < keep; ++s) {
            const int local = q - keep + s;        // row of this step, or (negative) of the old state
            v[s] = local >= 0 ? u[static_cast<size_t>(first + local) * in_stride + c]
                              : st[static_cast<size_t>(keep + local) * C + c];
        }
        for (int s = 0; s < keep; ++s) st[static_cast<size_t>(s) * C + c] = v[s];
    }
}

// ---------------------------- rotation of neighbouring pairs + unit norm + cache write
// A row of `qkv` holds nq query heads and nkv key heads of `hd` elements and nkv value heads of
// `vd` elements.  For every query and key head: entries (2i, 2i+1), 2i+1 < rot, of the token at
// position p turn by p * inv_freq[i]; then (unit_norm) the head is divided by its root mean
// square over hd (eps inside the root).  Queries are written back in place; keys and values go to
// their cache slots [pages, nkv, page_size, hd | vd] (and stay in `qkv` as they were).
// One CTA per token, one warp per head in turn; hd <= 256.
template <typename T>
__global__ void rotary_pairs_store_kernel(T* __restrict__ qkv, long long stride,
                                          const int* __restrict__ positions,
                                          const double* __restrict__ inv_freq, int nq, int nkv, int hd,
                                          int vd, int rot, int unit_norm, float eps,
                                          const int* __restrict__ slot_map, T* __restrict__ kcache,
                                          T* __restrict__ vcache, int page_size) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    T* row = qkv + static_cast<size_t>(t) * stride;
    // The angle position * frequency is formed in float64 and brought into [-pi, pi] there: in
    // float32 its rounding grows with the position (half an ulp of an angle of a thousand radians
    // is 3e-5, which a peaked softmax turns into an error of that relative size); sine and cosine
    // of the reduced angle are float32.
    const double pos = static_cast<double>(positions[t]);
    const int slot = slot_map != nullptr ? slot_map[t] : -1;
    const size_t page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
    for (int head = blockIdx.y * nwarps + warp; head < nq + nkv; head += nwarps * gridDim.y) {
        T* x = row + static_cast<size_t>(head) * hd;
        // a lane owns the pairs (2 i, 2 i + 1), i = lane + 32 j: one sine and cosine per pair; an
        // odd width's last element is a pair whose second half does not exist
        float va[4], vb[4];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = 2 * (lane + 32 * j);
            va[j] = vb[j] = 0.f;
            if (e < hd) {
                float a = to_float(x[e]);
                float b = e + 1 < hd ? to_float(x[e + 1]) : 0.f;
                if (e + 1 < rot) {
                    float sn, cs;
                    double angle = pos * inv_freq[e >> 1];
                    angle -= 6.283185307179586476925286766559 * rint(angle * 0.15915494309189533576888376337251);
                    sincosf(static_cast<float>(angle), &sn, &cs);
                    const float ra = fmaf(a, cs, -(b * sn)), rb = fmaf(b, cs, a * sn);
                    a = ra;
                    b = rb;
                }
                va[j] = a;
                vb[j] = b;
                ss = fmaf(a, a, fmaf(b, b, ss));
            }
        }
        ss = warp_sum(ss);         // also orders the reads of x before the writes below
        const float r = unit_norm ? 1.0f / sqrtf(ss / static_cast<float>(hd) + eps) : 1.0f;
        T* dst = nullptr;
        if (head < nq) dst = x;
        else if (slot >= 0) dst = kcache + ((page * nkv + (head - nq)) * page_size + off) * hd;
        if (dst != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int e = 2 * (lane + 32 * j);
                if (e < hd) {
                    dst[e] = from_float<T>(va[j] * r);
                    if (e + 1 < hd) dst[e + 1] = from_float<T>(vb[j] * r);
                }
            }
        }
    }
    if (slot >= 0 && blockIdx.y == 0) {
        const T* vrow = row + static_cast<size_t>(nq + nkv) * hd;
        for (int g = 0; g < nkv; ++g) {
            T* dst = vcache + ((page * nkv + g) * page_size + off) * vd;
            for (int e = threadIdx.x; e < vd; e += blockDim.x) dst[e] = vrow[static_cast<size_t>(g) * vd + e];
        }
    }
}

// ---------------------------------------------------------------- sigmoid gate
// x[t, c] *= sigmoid(g[t, c]); g's rows lie `g_stride` elements apart.
template <typename T>
__global__ void sigmoid_gate_mul_kernel(T* __restrict__ x, const T* __restrict__ g, long long g_stride,
                                        int C, long long n, int vec4) {
    pdl_launch_dependents();
    pdl_wait();
    if (vec4) {
        for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n;
             i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
            const long long t = i / C;
            const int c = static_cast<int>(i - t * C);
            const F4 z = load4(g + t * g_stride + c);
            F4 v = load4(x + i);
#pragma unroll
            for (int e = 0; e < 4; ++e) v.v[e] = v.v[e] / (1.0f + expf(-z.v[e]));
            store4(x + i, v);
        }
        return;
    }
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long t = i / C;
        const int c = static_cast<int>(i - t * C);
        const float z = to_float(g[t * g_stride + c]);
        x[i] = from_float<T>(to_float(x[i]) / (1.0f + expf(-z)));
    }
}

// ---------------------------------------------------------------- soft cap
// x = cap * tanh(x / cap), in place.
__global__ void softcap_kernel(float* __restrict__ x, float cap, long long n) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

// ------------------------------------------------------- state-space recurrence
// Per request r, head h (group g = h / (heads / groups)) and column p of the head, with a state
// M [N, P] float32 in the request's slot (stored [P, N]: a lane's rows n lie side by side):
//   dt = softplus(dt_raw[t, h] + dt_bias[h]);  M <- exp(-exp(a_log[h]) dt) M + (dt B_t) x_t^T;
//   y[t, h, p] = sum_n M[n, p] C_t[n] + D[h] x_t[p].
// x, B, C are columns [0, heads*P), then groups*N, then groups*N of the rows of `xbc`.
// A CTA owns kScanCols columns of one head of one request and walks through the request's rows
// of this step; a warp owns kScanColsPerWarp columns, a lane the state rows n = lane + 32 j.
// Rows are staged kScanBlock at a time in shared memory (B, C, the CTA's x columns, dt and the
// decay, each computed once), the next block's loads in flight while this one is worked on.
// The sum over n is taken in a fixed order (j, then lanes), so y does not depend on how the rows were cut.
// Index arithmetic of the staging is done once per thread, not per element.
constexpr int kScanWarps = 4;
constexpr int kScanColsPerWarp = 4;
constexpr int kScanCols = kScanWarps * kScanColsPerWarp;
constexpr int kScanBlock = 8;
constexpr int kScanThreads = kScanWarps * 32;

__device__ __forceinline__ float softplus_f(float z) {
    return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f);
}

template <typename T, int NPL>
__global__ void __launch_bounds__(kScanThreads)
ssm_scan_kernel(const T* __restrict__ xbc, long long x_stride, const T* __restrict__ dt_raw,
                long long dt_stride, const float* __restrict__ dt_bias,
                const float* __restrict__ a_log, const float* __restrict__ Dskip,
                float* __restrict__ state, const int* __restrict__ cu_q,
                const int* __restrict__ state_slot, float* __restrict__ y, int heads, int groups,
                int N, int P) {
    extern __shared__ float stage[];                       // [2][kScanBlock][row_f]
    // column slots of a staged row that one thread fetches: e = tid + c * kScanThreads < 2 N + kScanCols
    constexpr int kSlots = (64 * NPL + kScanCols + kScanThreads - 1) / kScanThreads;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta_p0 = blockIdx.z * kScanCols;
    const int p0 = cta_p0 + warp * kScanColsPerWarp;
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const int row_f = 2 * N + kScanCols + 2;               // B, C, x columns, dt, decay
    const int n_stage = kScanBlock * row_f;
    float* st = state + (static_cast<size_t>(state_slot[r]) * heads + h) * N * P;
    float m[NPL][kScanColsPerWarp];
#pragma unroll
    for (int j = 0; j < NPL; ++j)
#pragma unroll
        for (int i = 0; i < kScanColsPerWarp; ++i) {
            const int n = lane + 32 * j, p = p0 + i;
            m[j][i] = (n < N && p < P) ? st[static_cast<size_t>(p) * N + n] : 0.f;
        }
    const float rate = expf(a_log[h]), bias = dt_bias[h], skip = Dskip[h];
    const int first = cu_q[r], last = cu_q[r + 1];

    // where this thread's column slots lie in a row of xbc (-1: nothing to fetch, zero is staged)
    int col_off[kSlots];
#pragma unroll
    for (int c = 0; c < kSlots; ++c) {
        const int e = tid + c * kScanThreads;
        int off = -1;
        if (e < N) off = inner + g * N + e;
        else if (e < 2 * N) off = inner + (groups + g) * N + (e - N);
        else if (e < 2 * N + kScanCols && cta_p0 + (e - 2 * N) < P) off = h * P + cta_p0 + (e - 2 * N);
        col_off[c] = off;
    }
    T raw[kSlots][kScanBlock];
    T raw_dt = from_float<T>(0.f);
    // the loads of a block are all in flight at once; they become float32 (and dt, decay) when
    // they are put into shared memory, one block later
    auto issue = [&](int t0) {
#pragma unroll
        for (int tok = 0; tok < kScanBlock; ++tok) {
            if (t0 + tok < last) {
                const T* row = xbc + static_cast<size_t>(t0 + tok) * x_stride;
#pragma unroll
                for (int c = 0; c < kSlots; ++c)
                    if (col_off[c] >= 0) raw[c][tok] = row[col_off[c]];
            }
        }
        if (tid < kScanBlock && t0 + tid < last)
            raw_dt = dt_raw[static_cast<size_t>(t0 + tid) * dt_stride + h];
    };
    auto stash = [&](float* cur) {
#pragma unroll
        for (int c = 0; c < kSlots; ++c) {
            const int e = tid + c * kScanThreads;
            if (e < 2 * N + kScanCols) {
#pragma unroll
                for (int tok = 0; tok < kScanBlock; ++tok)
                    cur[tok * row_f + e] = col_off[c] >= 0 ? to_float(raw[c][tok]) : 0.f;
            }
        }
        if (tid < kScanBlock) {
            const float dt = softplus_f(to_float(raw_dt) + bias);
            cur[tid * row_f + 2 * N + kScanCols] = dt;
            cur[tid * row_f + 2 * N + kScanCols + 1] = expf(-rate * dt);
        }
    };
    // A lane's partial sums over its own state rows go to shared memory, [row of the block][column]
    // [lane] with rows of 33 floats; after the block's rows, lane 4 t + c adds up the 32 partial
    // sums of (row t, column c) in lane order.  The loop over rows then carries nothing but the
    // state itself, one multiply-add deep, so consecutive rows overlap.
    static_assert(kScanBlock * kScanColsPerWarp == 32, "one (row, column) pair per lane");
    float* part = stage + 2 * n_stage + warp * (32 * 33);
    if (first < last) issue(first);
    int buf = 0;
    for (int t0 = first; t0 < last; t0 += kScanBlock) {
        float* cur = stage + buf * n_stage;
        stash(cur);
        __syncthreads();
        if (t0 + kScanBlock < last) issue(t0 + kScanBlock);
        const int n_tok = min(kScanBlock, last - t0);
        if (p0 < P) {
            for (int tok = 0; tok < n_tok; ++tok) {
                const float* row = cur + tok * row_f;
                const float dt = row[2 * N + kScanCols], decay = row[2 * N + kScanCols + 1];
                float xv[kScanColsPerWarp], acc[kScanColsPerWarp];
#pragma unroll
                for (int i = 0; i < kScanColsPerWarp; ++i) {
                    xv[i] = row[2 * N + warp * kScanColsPerWarp + i];
                    acc[i] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < NPL; ++j) {
                    const int n = lane + 32 * j;
                    const float bn = n < N ? row[n] * dt : 0.f;
                    const float cn = n < N ? row[N + n] : 0.f;
#pragma unroll
                    for (int i = 0; i < kScanColsPerWarp; ++i) {
                        m[j][i] = fmaf(decay, m[j][i], bn * xv[i]);
                        acc[i] = fmaf(m[j][i], cn, acc[i]);
                    }
                }
#pragma unroll
                for (int i = 0; i < kScanColsPerWarp; ++i)
                    part[(tok * kScanColsPerWarp + i) * 33 + lane] = acc[i];
            }
            __syncwarp();
            const int tok = lane / kScanColsPerWarp, col = lane % kScanColsPerWarp;
            if (tok < n_tok && p0 + col < P) {
                const float* mine = part + lane * 33;
                float v = 0.f;
#pragma unroll
                for (int k = 0; k < 32; ++k) v += mine[k];
                y[static_cast<size_t>(t0 + tok) * inner + static_cast<size_t>(h) * P + p0 + col] =
                    fmaf(skip, cur[tok * row_f + 2 * N + warp * kScanColsPerWarp + col], v);
            }
            __syncwarp();
        }
        buf ^= 1;       // the block after the next overwrites this buffer only behind the next barrier
    }
#pragma unroll
    for (int j = 0; j < NPL; ++j)
#pragma unroll
        for (int i = 0; i < kScanColsPerWarp; ++i) {
            const int n = lane + 32 * j, p = p0 + i;
            if (n < N && p < P) st[static_cast<size_t>(p) * N + n] = m[j][i];
        }
}

// ------------------------------------------------------- gated group RMS norm
// v = y[t] * silu(z[t]) (z's rows `z_stride` apart); the C columns in `groups` equal parts, each
// divided by its own root mean square; out = that * weight.  One CTA per (token, part).
template <typename T>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ z,
                                           long long z_stride, const void* __restrict__ weight,
                                           int w_dtype, float eps, T* __restrict__ out, int C,
                                           int groups, int vec4) {
    extern __shared__ __align__(16) float vals[];          // the part's gated values
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, part = blockIdx.y;
    const int n = C / groups, c0 = part * n;
    const float* yr = y + static_cast<size_t>(t) * C + c0;
    const T* zr = z + static_cast<size_t>(t) * z_stride + c0;
    T* o = out + static_cast<size_t>(t) * C + c0;
    float ss = 0.f;
    if (vec4) {
        for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
            const F4 zz = load4(zr + i);
            F4 v = load4(yr + i);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                v.v[e] *= zz.v[e] / (1.0f + expf(-zz.v[e]));
                ss = fmaf(v.v[e], v.v[e], ss);
            }
            store4(vals + i, v);
        }
        ss = block_sum(ss, scratch);
        const float r = 1.0f / sqrtf(ss / static_cast<float>(n) + eps);
        for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
            const F4 w = load4_any(weight, w_dtype, c0 + i);
            F4 v = load4(vals + i);
#pragma unroll
            for (int e = 0; e < 4; ++e) v.v[e] = v.v[e] * r * w.v[e];
            store4(o + i, v);
        }
        return;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float zz = to_float(zr[i]);
        const float v = yr[i] * (zz / (1.0f + expf(-zz)));
        vals[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / static_cast<float>(n) + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        o[i] = from_float<T>(vals[i] * r * load_as_float(weight, w_dtype, c0 + i));
}

}  // namespace somi

using namespace somi;

static inline int block_for(int n) { return min(256, max(32, ((n + 31) / 32) * 32)); }

SOMI_API int somi_embed_scaled(const int* ids, const void* table, int dtype, float scale, float* out,
                               int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (dtype == SOMI_F32)
        launch_pdl(embed_scaled_kernel<float>, dim3(T), dim3(block_for(H)), 0, stream, ids,
                   static_cast<const float*>(table), scale, out, H);
    else
        launch_pdl(embed_scaled_kernel<__nv_bfloat16>, dim3(T), dim3(block_for(H)), 0, stream, ids,
                   static_cast<const __nv_bfloat16*>(table), scale, out, H);
    return launch_status();
}

SOMI_API int somi_add_normed_rmsnorm(float* residual, const void* delta, int delta_dtype, int splits,
                                     long long split_stride, const void* weight_b, int wb_dtype,
                                     float eps_b, const void* weight, int w_dtype, float eps,
                                     void* out, int out_dtype, const int* rows, int n_out, int H,
                                     int write_back, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (splits > 1 && delta_dtype != SOMI_F32) return SOMI_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * H;
    if (smem > 200 * 1024) return SOMI_ERR_UNSUPPORTED;
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const int vec4 = (H & 3) == 0 && aligned(residual) && aligned(delta) && aligned(weight_b) &&
                     aligned(weight) && aligned(out) && (split_stride & 3) == 0;
    // few rows (a decode step): a thread per four columns; many rows: a quarter of that
    const int threads = vec4 ? min(1024, max(32, (((n_out <= 512 ? H / 4 : H / 16) + 31) / 32) * 32))
                             : block_for(H / 2);
#define SOMI_LAUNCH_SN(TD, TO)                                                                    \
    do {                                                                                          \
        if (smem > 48 * 1024)                                                                     \
            cudaFuncSetAttribute(add_normed_rmsnorm_kernel<TD, TO>,                               \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
        launch_pdl(add_normed_rmsnorm_kernel<TD, TO>, dim3(n_out), dim3(threads), smem, stream,   \
                   residual, static_cast<const TD*>(delta), splits, split_stride, weight_b,       \
                   wb_dtype, eps_b, weight, w_dtype, eps, static_cast<TO*>(out), rows, H,         \
                   write_back, vec4);                                                             \
    } while (0)
    if (delta_dtype == SOMI_F32 && out_dtype == SOMI_F32) SOMI_LAUNCH_SN(float, float);
    else if (delta_dtype == SOMI_F32) SOMI_LAUNCH_SN(float, __nv_bfloat16);
    else if (out_dtype == SOMI_F32) SOMI_LAUNCH_SN(__nv_bfloat16, float);
    else SOMI_LAUNCH_SN(__nv_bfloat16, __nv_bfloat16);
#undef SOMI_LAUNCH_SN
    return launch_status();
}

SOMI_API int somi_causal_conv_max_taps() { return kConvMaxTaps; }

// u: [T, in_stride] (C channels from the pointer on); w: float32 [taps, C]; bias: float32 [C] or
// null; state: [slots, taps - 1, C] of u's dtype, moved on by this step's rows; out: [T, out_stride].
SOMI_API int somi_causal_conv(const void* u, int dtype, long long in_stride, const float* w,
                              const float* bias, void* state, const int* cu_q,
                              const int* token_request, const int* state_slot, void* out,
                              long long out_stride, int T, int R, int C, int taps, int act,
                              int add_input, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (taps < 1 || taps > kConvMaxTaps || R <= 0 || C <= 0) return SOMI_ERR_UNSUPPORTED;
    const int tb = min(256, ((C + 31) / 32) * 32);
    const int chunks = max(1, min(64, (C + tb - 1) / tb));
    // four channels a thread where every row starts on a vector boundary (16 bytes of float32, 8 of
    // bfloat16)
    const uintptr_t mask = dtype == SOMI_F32 ? 15 : 7;
    const int vec4 = (C & 3) == 0 && (in_stride & 3) == 0 && (out_stride & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(out) |
                       reinterpret_cast<uintptr_t>(state)) & mask) == 0 &&
                     ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(bias)) & 15) == 0;
    const int per = vec4 ? 4 : 1;
#define SOMI_LAUNCH_CONV(TT)                                                                     \
    do {                                                                                         \
        launch_pdl(causal_conv_kernel<TT>,                                                       \
                   dim3((T + 3) / 4, max(1, min(T <= 64 ? 128 : 8, (C / per + 63) / 64))),       \
                   dim3(64, 4), 0, stream, static_cast<const TT*>(u), in_stride, w, bias,        \
                   static_cast<const TT*>(state), cu_q, token_request, state_slot,               \
                   static_cast<TT*>(out), out_stride, C, taps, act, add_input, T, vec4);         \
        if (taps > 1)                                                                            \
            launch_pdl(causal_conv_state_kernel<TT>, dim3(R, chunks), dim3(tb), 0, stream,       \
                       static_cast<const TT*>(u), in_stride, static_cast<TT*>(state), cu_q,      \
                       state_slot, C, taps);                                                     \
    } while (0)
    if (dtype == SOMI_F32) SOMI_LAUNCH_CONV(float);
    else SOMI_LAUNCH_CONV(__nv_bfloat16);
#undef SOMI_LAUNCH_CONV
    return launch_status();
}

SOMI_API int somi_rotary_pairs_store(void* qkv, int dtype, long long stride, const int* positions,
                                     const double* inv_freq, int T, int nq, int nkv, int hd, int vd,
                                     int rot, int unit_norm, float eps, const int* slot_map,
                                     void* kcache, void* vcache, int page_size, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > 256 || vd <= 0 || rot < 0 || rot > hd || (rot & 1) || nq <= 0 || nkv <= 0)
        return SOMI_ERR_UNSUPPORTED;
    const int threads = 32 * min(8, nq + nkv);
    // few tokens: a warp per head, so that a step of single tokens still fills the SMs
    const dim3 grid(T, T <= 256 ? (nq + nkv + 7) / 8 : 1);
    if (dtype == SOMI_F32)
        launch_pdl(rotary_pairs_store_kernel<float>, grid, dim3(threads), 0, stream,
                   static_cast<float*>(qkv), stride, positions, inv_freq, nq, nkv, hd, vd, rot,
                   unit_norm, eps, slot_map, static_cast<float*>(kcache),
                   static_cast<float*>(vcache), page_size);
    else
        launch_pdl(rotary_pairs_store_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream,
                   static_cast<__nv_bfloat16*>(qkv), stride, positions, inv_freq, nq, nkv, hd, vd,
                   rot, unit_norm, eps, slot_map, static_cast<__nv_bfloat16*>(kcache),
                   static_cast<__nv_bfloat16*>(vcache), page_size);
    return launch_status();
}

SOMI_API int somi_sigmoid_gate_mul(void* x, const void* g, int dtype, long long g_stride, long long T,
                                   int C, cudaStream_t stream) {
    const long long n = T * C;
    if (n <= 0) return 0;
    const uintptr_t mask = dtype == SOMI_F32 ? 15 : 7;
    const int vec4 = (C & 3) == 0 && (g_stride & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g)) & mask) == 0;
    const long long work = vec4 ? n / 4 : n;
    const int blocks = static_cast<int>(((work + 255) / 256) < 148LL * 16 ? ((work + 255) / 256) : 148LL * 16);
    if (dtype == SOMI_F32)
        launch_pdl(sigmoid_gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<float*>(x), static_cast<const float*>(g), g_stride, C, n, vec4);
    else
        launch_pdl(sigmoid_gate_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                   static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(g), g_stride, C, n,
                   vec4);
    return launch_status();
}

SOMI_API int somi_softcap(float* x, float cap, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return SOMI_ERR_UNSUPPORTED;
    const int blocks = static_cast<int>(((n + 255) / 256) < 148LL * 16 ? ((n + 255) / 256) : 148LL * 16);
    launch_pdl(softcap_kernel, dim3(blocks), dim3(256), 0, stream, x, cap, n);
    return launch_status();
}

SOMI_API int somi_ssm_scan_max_state() { return 512; }

SOMI_API int somi_ssm_scan(const void* xbc, int dtype, long long x_stride, const void* dt_raw,
                           long long dt_stride, const float* dt_bias, const float* a_log,
                           const float* Dskip, float* state, const int* cu_q, const int* state_slot,
                           float* y, int R, int heads, int groups, int N, int P,
                           cudaStream_t stream) {
    if (R <= 0) return 0;
    if (N <= 0 || N > 512 || P <= 0 || heads <= 0 || groups <= 0 || heads % groups)
        return SOMI_ERR_UNSUPPORTED;
    dim3 grid(R, heads, (P + kScanCols - 1) / kScanCols);
    const int npl = (N + 31) / 32;
    const size_t smem = sizeof(float) * (2 * kScanBlock * (2 * N + kScanCols + 2) + kScanWarps * 32 * 33);
#define SOMI_LAUNCH_SCAN(TT, NPL)                                                                \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(ssm_scan_kernel<TT, NPL>,                                       \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        launch_pdl(ssm_scan_kernel<TT, NPL>, grid, dim3(kScanThreads), smem, stream,             \
                   static_cast<const TT*>(xbc), x_stride, static_cast<const TT*>(dt_raw),        \
                   dt_stride, dt_bias, a_log, Dskip, state, cu_q, state_slot, y, heads, groups,  \
                   N, P);                                                                        \
    } while (0)
#define SOMI_SCAN_BY_N(TT)                                                                       \
    do {                                                                                         \
        if (npl <= 1) SOMI_LAUNCH_SCAN(TT, 1);                                                   \
        else if (npl <= 2) SOMI_LAUNCH_SCAN(TT, 2);                                              \
        else if (npl <= 4) SOMI_LAUNCH_SCAN(TT, 4);                                              \
        else if (npl <= 8) SOMI_LAUNCH_SCAN(TT, 8);                                              \
        else SOMI_LAUNCH_SCAN(TT, 16);                                                           \
    } while (0)
    if (dtype == SOMI_F32) SOMI_SCAN_BY_N(float);
    else SOMI_SCAN_BY_N(__nv_bfloat16);
#undef SOMI_SCAN_BY_N
#undef SOMI_LAUNCH_SCAN
    return launch_status();
}

SOMI_API int somi_gated_group_rmsnorm(const float* y, const void* z, int dtype, long long z_stride,
                                      const void* weight, int w_dtype, float eps, void* out, int T,
                                      int C, int groups, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (groups <= 0 || C % groups) return SOMI_ERR_UNSUPPORTED;
    const int n = C / groups;
    const size_t smem = sizeof(float) * n;
    if (smem > 200 * 1024) return SOMI_ERR_UNSUPPORTED;
    const uintptr_t mask = dtype == SOMI_F32 ? 15 : 7;
    const int vec4 = (n & 3) == 0 && (z_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(weight) & 15) == 0 &&
                     ((reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(out)) & mask) == 0;
    const int threads = block_for(vec4 ? n / 4 : n / 2);
#define SOMI_LAUNCH_GGN(TT)                                                                       \
    do {                                                                                          \
        if (smem > 48 * 1024)                                                                     \
            cudaFuncSetAttribute(gated_group_rmsnorm_kernel<TT>,                                  \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
        launch_pdl(gated_group_rmsnorm_kernel<TT>, dim3(T, groups), dim3(threads), smem, stream, y, \
                   static_cast<const TT*>(z), z_stride, weight, w_dtype, eps,                     \
                   static_cast<TT*>(out), C, groups, vec4);                                       \
    } while (0)
    if (dtype == SOMI_F32) SOMI_LAUNCH_GGN(float);
    else SOMI_LAUNCH_GGN(__nv_bfloat16);
#undef SOMI_LAUNCH_GGN
    return launch_status();
}
