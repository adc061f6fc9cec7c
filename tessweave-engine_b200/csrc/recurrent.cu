// Gated linear recurrences with a state of fixed size per request.
//
// minGRU: the gates read only the current token, so a request's rows form the first-order recurrence
//   z_t = sigmoid(pz_t + bz)         u_t = px_t + bx        c_t = u_t + 1/2 (u_t >= 0), sigmoid(u_t) (u_t < 0)
//   S_t = (1 - z_t) S_{t-1} + z_t c_t                        element by element, fp32, S_{-1} = the request's state
//   out_t = T(S_t * silu(pg_t))
// with pz | px | pg the three column blocks of one projection row.  The state slot of a request is read at
// the first row of a step and written back after its last, so a request may be cut into steps anywhere.
// Everything behind the projection is fp32.
#include "common.cuh"

#define TW_SCAN_THREADS 128

__device__ __forceinline__ float tw_sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }
// the segmented kernel's gates: accurate in float32 runs; in bfloat16 runs, whose pre-activations carry 8 bits,
// the hardware's exponential and reciprocal (fp32 all the same, a few units in the last place)
template <typename T> __device__ __forceinline__ float tw_gate_sigmoid(float x);
template <> __device__ __forceinline__ float tw_gate_sigmoid<float>(float x) { return 1.0f / (1.0f + expf(-x)); }
template <> __device__ __forceinline__ float tw_gate_sigmoid<__nv_bfloat16>(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// Short portions and single tokens: one thread per (request, channel) walks the request's rows of this step in order.
template <typename T>
__global__ void __launch_bounds__(TW_SCAN_THREADS)
mingru_scan_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ proj, int proj_stride,
                   const float* __restrict__ bias_z, const float* __restrict__ bias_x, float* __restrict__ state,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                   const int* __restrict__ seq_q_len, int width, int write_state) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int s = blockIdx.y;
    const int ch = blockIdx.x * TW_SCAN_THREADS + threadIdx.x;
    const int len = seq_q_len[s];
    if (ch >= width || len <= 0) return;
    const int start = seq_q_start[s];
    float* slot = state + (size_t)seq_slot[s] * width;
    float S = slot[ch];
    const float bz = bias_z ? bias_z[ch] : 0.f, bx = bias_x ? bias_x[ch] : 0.f;
    for (int t = 0; t < len; ++t) {
        const T* row = proj + (size_t)(start + t) * proj_stride;
        const float z = tw_sigmoidf(tw_to_float(row[ch]) + bz);
        const float u = tw_to_float(row[width + ch]) + bx;
        const float g = tw_to_float(row[2 * width + ch]);
        const float c = u >= 0.f ? u + 0.5f : tw_sigmoidf(u);
        S = (1.0f - z) * S + z * c;
        out[(size_t)(start + t) * out_stride + ch] = tw_from_float<T>(S * (g * tw_sigmoidf(g)));
    }
    if (write_state) slot[ch] = S;
}

// Long portions: a block of 32 warps takes 32 channels of one request; warp w walks the w-th segment of the
// request's rows from a zero state and keeps only (A, B) with S_end = A * S_in + B; the segments are chained
// in shared memory; then every warp walks its segment again from its true S_in and writes the rows.  The
// second pass finds its operands in L2.  Sums are formed in the order of the rows inside a segment and in the
// order of the segments between them, whatever the hardware does.
#define TW_SCAN_SEGMENTS 32

template <typename T>
__global__ void __launch_bounds__(32 * TW_SCAN_SEGMENTS)
mingru_scan_segments_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ proj, int proj_stride,
                            const float* __restrict__ bias_z, const float* __restrict__ bias_x, float* __restrict__ state,
                            const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                            const int* __restrict__ seq_q_len, int width, int write_state) {
    __shared__ float sA[TW_SCAN_SEGMENTS][33], sB[TW_SCAN_SEGMENTS][33];
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int s = blockIdx.y;
    const int lane = threadIdx.x & 31, seg = threadIdx.x >> 5;
    const int ch = blockIdx.x * 32 + lane;
    const int len = seq_q_len[s];
    if (len <= 0) return;
    const bool live = ch < width;
    const int start = seq_q_start[s];
    const int per = (len + TW_SCAN_SEGMENTS - 1) / TW_SCAN_SEGMENTS;
    const int t0 = min(len, seg * per), t1 = min(len, t0 + per);
    const float bz = (live && bias_z) ? bias_z[ch] : 0.f, bx = (live && bias_x) ? bias_x[ch] : 0.f;
    float A = 1.f, B = 0.f;
    if (live) {
        // the loads and gates of a row do not depend on the row before: eight rows at a time, so that their
        // round trips to memory overlap, then the eight steps of the recurrence in order
        int t = t0;
        for (; t + 8 <= t1; t += 8) {
            float zs[8], cs[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const T* row = proj + (size_t)(start + t + k) * proj_stride;
                zs[k] = tw_to_float(row[ch]);
                cs[k] = tw_to_float(row[width + ch]);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float z = tw_gate_sigmoid<T>(zs[k] + bz);
                const float u = cs[k] + bx;
                const float c = u >= 0.f ? u + 0.5f : tw_gate_sigmoid<T>(u);
                A *= 1.0f - z;
                B = (1.0f - z) * B + z * c;
            }
        }
        for (; t < t1; ++t) {
            const T* row = proj + (size_t)(start + t) * proj_stride;
            const float z = tw_gate_sigmoid<T>(tw_to_float(row[ch]) + bz);
            const float u = tw_to_float(row[width + ch]) + bx;
            const float c = u >= 0.f ? u + 0.5f : tw_gate_sigmoid<T>(u);
            A *= 1.0f - z;
            B = (1.0f - z) * B + z * c;
        }
    }
    sA[seg][lane] = A;
    sB[seg][lane] = B;
    __syncthreads();
    float* slot = state + (size_t)seq_slot[s] * width;
    if (seg == 0 && live) {
        float S = slot[ch];
        for (int k = 0; k < TW_SCAN_SEGMENTS; ++k) {
            const float a = sA[k][lane], b = sB[k][lane];
            sA[k][lane] = S;                 // what segment k starts from
            S = a * S + b;
        }
        if (write_state) slot[ch] = S;
    }
    __syncthreads();
    if (!live) return;
    float S = sA[seg][lane];
    int t = t0;
    for (; t + 8 <= t1; t += 8) {
        float zs[8], cs[8], gs[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const T* row = proj + (size_t)(start + t + k) * proj_stride;
            zs[k] = tw_to_float(row[ch]);
            cs[k] = tw_to_float(row[width + ch]);
            gs[k] = tw_to_float(row[2 * width + ch]);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float z = tw_gate_sigmoid<T>(zs[k] + bz);
            const float u = cs[k] + bx;
            const float c = u >= 0.f ? u + 0.5f : tw_gate_sigmoid<T>(u);
            S = (1.0f - z) * S + z * c;
            out[(size_t)(start + t + k) * out_stride + ch] = tw_from_float<T>(S * (gs[k] * tw_gate_sigmoid<T>(gs[k])));
        }
    }
    for (; t < t1; ++t) {
        const T* row = proj + (size_t)(start + t) * proj_stride;
        const float z = tw_gate_sigmoid<T>(tw_to_float(row[ch]) + bz);
        const float u = tw_to_float(row[width + ch]) + bx;
        const float g = tw_to_float(row[2 * width + ch]);
        const float c = u >= 0.f ? u + 0.5f : tw_gate_sigmoid<T>(u);
        S = (1.0f - z) * S + z * c;
        out[(size_t)(start + t) * out_stride + ch] = tw_from_float<T>(S * (g * tw_gate_sigmoid<T>(g)));
    }
}

TW_EXPORT int tw_mingru_scan(void* out, int out_stride, const void* proj, int proj_stride, const float* bias_z,
                             const float* bias_x, float* state, const int* seq_slot, const int* seq_q_start,
                             const int* seq_q_len, int n_seqs, int max_q_len, int width, int write_state, int dtype,
                             cudaStream_t stream) {
    if (n_seqs <= 0 || width <= 0) return 0;
    if (max_q_len > 2 * TW_SCAN_SEGMENTS) {
        const dim3 grid((width + 31) / 32, n_seqs);
        if (dtype == TW_F32)
            return tw_launch(mingru_scan_segments_kernel<float>, grid, dim3(32 * TW_SCAN_SEGMENTS), 0, stream, 1, (float*)out,
                             out_stride, (const float*)proj, proj_stride, bias_z, bias_x, state, seq_slot, seq_q_start,
                             seq_q_len, width, write_state);
        return tw_launch(mingru_scan_segments_kernel<__nv_bfloat16>, grid, dim3(32 * TW_SCAN_SEGMENTS), 0, stream, 1,
                         (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)proj, proj_stride, bias_z, bias_x, state,
                         seq_slot, seq_q_start, seq_q_len, width, write_state);
    }
    const dim3 grid((width + TW_SCAN_THREADS - 1) / TW_SCAN_THREADS, n_seqs);
    if (dtype == TW_F32)
        return tw_launch(mingru_scan_kernel<float>, grid, dim3(TW_SCAN_THREADS), 0, stream, 1, (float*)out, out_stride,
                         (const float*)proj, proj_stride, bias_z, bias_x, state, seq_slot, seq_q_start, seq_q_len, width,
                         write_state);
    return tw_launch(mingru_scan_kernel<__nv_bfloat16>, grid, dim3(TW_SCAN_THREADS), 0, stream, 1, (__nv_bfloat16*)out,
                     out_stride, (const __nv_bfloat16*)proj, proj_stride, bias_z, bias_x, state, seq_slot, seq_q_start,
                     seq_q_len, width, write_state);
}

// ---------------------------------------------------------------------------
// What follows a recurrence: per (row, head)  o = raw / den (where a denominator is given),
// y = o / sqrt(mean(o^2) + eps) * weight * act(gate), rounded to the activation type.  One warp per (row, head).
// act: 0 none, 1 silu, 2 sigmoid.  Everything in fp32.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(T* __restrict__ out, int out_stride, const float* __restrict__ raw, const float* __restrict__ den,
                      const float* __restrict__ weight, const T* __restrict__ gate, int gate_stride, int act, float eps,
                      int rows, int H, int Dv) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= rows * H) return;
    const int row = item / H, h = item - row * H;
    const float* r = raw + (size_t)row * H * Dv + (size_t)h * Dv;
    const float inv_den = den ? 1.0f / den[(size_t)row * H + h] : 1.0f;
    float ss = 0.f;
    for (int d = lane; d < Dv; d += 32) {
        const float o = r[d] * inv_den;
        ss += o * o;
    }
    ss = tw_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)Dv + eps);
    for (int d = lane; d < Dv; d += 32) {
        float y = r[d] * inv_den * inv;
        if (weight) y *= weight[h * Dv + d];
        if (act) {
            const float g = tw_to_float(gate[(size_t)row * gate_stride + h * Dv + d]);
            const float sg = 1.0f / (1.0f + expf(-g));
            y *= act == 1 ? g * sg : sg;
        }
        out[(size_t)row * out_stride + h * Dv + d] = tw_from_float<T>(y);
    }
}

TW_EXPORT int tw_head_norm_gate(void* out, int out_stride, const float* raw, const float* den, const float* weight,
                                const void* gate, int gate_stride, int act, float eps, int rows, int H, int Dv, int dtype,
                                cudaStream_t stream) {
    if (rows <= 0 || H <= 0) return 0;
    const dim3 grid((unsigned)(((size_t)rows * H + 3) / 4));
    if (dtype == TW_F32)
        return tw_launch(head_norm_gate_kernel<float>, grid, dim3(128), 0, stream, 1, (float*)out, out_stride, raw, den, weight,
                         (const float*)gate, gate_stride, act, eps, rows, H, Dv);
    return tw_launch(head_norm_gate_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, 1, (__nv_bfloat16*)out, out_stride, raw,
                     den, weight, (const __nv_bfloat16*)gate, gate_stride, act, eps, rows, H, Dv);
}

// ---------------------------------------------------------------------------
// Token shift: out[m][row] = h[row] + (h[row - 1] - h[row]) * mu[m] for `n_mix` blends of a row with the row
// before it in the same request.  A request's first row of a step takes the row the step before left in the
// request's state (zeros at the very first token).  fp32 arithmetic, rounded once.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
token_shift_mix_kernel(T* __restrict__ out, size_t mix_stride, const T* __restrict__ h, int h_stride,
                       const float* __restrict__ mu, const float* __restrict__ state, long long state_stride,
                       long long state_offset, const int* __restrict__ seq_of_token, const int* __restrict__ seq_slot,
                       const int* __restrict__ seq_q_start, int width, int n_mix) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int row = blockIdx.x;
    const int s = seq_of_token[row];
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float cur = 0.f, prev = 0.f;
        if (s >= 0) {
            cur = tw_to_float(h[(size_t)row * h_stride + c]);
            prev = row == seq_q_start[s] ? state[(size_t)seq_slot[s] * state_stride + state_offset + c]
                                         : tw_to_float(h[(size_t)(row - 1) * h_stride + c]);
        }
        for (int m = 0; m < n_mix; ++m)
            out[(size_t)m * mix_stride + (size_t)row * width + c] = tw_from_float<T>(cur + (prev - cur) * mu[(size_t)m * width + c]);
    }
}

// bf16 rows whose width is a multiple of 8: a thread blends eight neighbouring channels with 16-byte accesses.
__global__ void __launch_bounds__(512)
token_shift_mix_bf16x8_kernel(__nv_bfloat16* __restrict__ out, size_t mix_stride, const __nv_bfloat16* __restrict__ h, int h_stride,
                              const float* __restrict__ mu, const float* __restrict__ state, long long state_stride,
                              long long state_offset, const int* __restrict__ seq_of_token, const int* __restrict__ seq_slot,
                              const int* __restrict__ seq_q_start, int width, int n_mix) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int row = blockIdx.x;
    const int s = seq_of_token[row];
    for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
        float cur[8], prev[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) cur[e] = prev[e] = 0.f;
        if (s >= 0) {
            const uint4 raw = *reinterpret_cast<const uint4*>(h + (size_t)row * h_stride + c);
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p2[e]); cur[2 * e] = f.x; cur[2 * e + 1] = f.y; }
            if (row == seq_q_start[s]) {
                const float* st = state + (size_t)seq_slot[s] * state_stride + state_offset + c;
#pragma unroll
                for (int e = 0; e < 8; ++e) prev[e] = st[e];
            } else {
                const uint4 rawp = *reinterpret_cast<const uint4*>(h + (size_t)(row - 1) * h_stride + c);
                const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&rawp);
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(q2[e]); prev[2 * e] = f.x; prev[2 * e + 1] = f.y; }
            }
        }
        for (int m = 0; m < n_mix; ++m) {
            const float* mr = mu + (size_t)m * width + c;
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e)
                o2[e] = __floats2bfloat162_rn(cur[2 * e] + (prev[2 * e] - cur[2 * e]) * mr[2 * e],
                                              cur[2 * e + 1] + (prev[2 * e + 1] - cur[2 * e + 1]) * mr[2 * e + 1]);
            *reinterpret_cast<uint4*>(out + (size_t)m * mix_stride + (size_t)row * width + c) = o;
        }
    }
}

TW_EXPORT int tw_token_shift_mix(void* out, long long mix_stride, const void* h, int h_stride, const float* mu,
                                 const float* state, long long state_stride, long long state_offset,
                                 const int* seq_of_token, const int* seq_slot, const int* seq_q_start, int rows, int width,
                                 int n_mix, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == TW_F32)
        return tw_launch(token_shift_mix_kernel<float>, dim3(rows), dim3(256), 0, stream, 1, (float*)out, (size_t)mix_stride,
                         (const float*)h, h_stride, mu, state, state_stride, state_offset, seq_of_token, seq_slot,
                         seq_q_start, width, n_mix);
    if ((width & 7) == 0 && (h_stride & 7) == 0 && (mix_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(h) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        const int threads = min(512, ((width / 8 + 31) / 32) * 32);
        return tw_launch(token_shift_mix_bf16x8_kernel, dim3(rows), dim3(threads), 0, stream, 1, (__nv_bfloat16*)out,
                         (size_t)mix_stride, (const __nv_bfloat16*)h, h_stride, mu, state, state_stride, state_offset,
                         seq_of_token, seq_slot, seq_q_start, width, n_mix);
    }
    return tw_launch(token_shift_mix_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, 1, (__nv_bfloat16*)out,
                     (size_t)mix_stride, (const __nv_bfloat16*)h, h_stride, mu, state, state_stride, state_offset,
                     seq_of_token, seq_slot, seq_q_start, width, n_mix);
}

// tanh of every element, in place (the activation between the two small matrices of a projected decay).
template <typename T>
__global__ void tanh_rows_kernel(T* __restrict__ x, size_t count) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) x[i] = tw_from_float<T>(tanhf(tw_to_float(x[i])));
}

TW_EXPORT int tw_tanh_rows(void* x, long long count, int dtype, cudaStream_t stream) {
    if (count <= 0) return 0;
    const dim3 grid((unsigned)((count + 255) / 256));
    if (dtype == TW_F32) return tw_launch(tanh_rows_kernel<float>, grid, dim3(256), 0, stream, 1, (float*)x, (size_t)count);
    return tw_launch(tanh_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, 1, (__nv_bfloat16*)x, (size_t)count);
}

// ---------------------------------------------------------------------------
// Short causal convolution over time, per channel, with silu, for the packed rows a recurrence reads:
//   y[t, c] = silu(sum_j w[c, j] x[t - (taps - 1) + j, c]),   the last tap is the row's own, zeros before a request's start.
// The taps - 1 rows before a request's first row of this step come from the request's state (fp32, channel-major:
// state[offset + c * (taps - 1) + j], j = 0 the oldest), which tw_short_conv_state moves on afterwards.  Behind the
// convolution the first `unit_heads` heads of `unit_dim` channels are scaled to unit length, x / sqrt(sum x^2 + unit_eps),
// the first `scaled_heads` of them also multiplied by `head_scale`.  One block per row; the result is fp32.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
short_conv_kernel(float* __restrict__ out, const T* __restrict__ x, int x_stride, const float* __restrict__ w, int taps,
                  float* __restrict__ state, long long state_stride, long long state_offset,
                  const int* __restrict__ seq_of_token, const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                  const int* __restrict__ seq_q_len, int move_single, int channels, int chunk, int unit_heads, int unit_dim,
                  int scaled_heads, float head_scale, float unit_eps) {
    extern __shared__ float sy[];        // [chunk]
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int row = blockIdx.x;
    const int s = seq_of_token[row];
    if (s < 0) return;
    // this block's channels: a whole number of unit heads, so that no head's sum of squares crosses blocks
    const int c0 = blockIdx.y * chunk, c1 = min(channels, c0 + chunk);
    const int r = row - seq_q_start[s];                  // rows of this request before this one in the step
    float* tail = state + (size_t)seq_slot[s] * state_stride + state_offset;
    // A request that brings one row has no other block that reads these channels of its state: the thread that read
    // them moves them on itself (the oldest input leaves, the row's own joins), and the step needs no second kernel.
    const bool move = move_single && seq_q_len[s] == 1 && taps > 1;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float acc = 0.f;
        float* tc = tail + (size_t)c * (taps - 1);
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;               // how many rows before this one
            const float xv = back <= r ? tw_to_float(x[(size_t)(row - back) * x_stride + c]) : tc[taps - 1 + r - back];
            acc += w[(size_t)c * taps + j] * xv;
            if (move && j > 0) tc[j - 1] = xv;           // r == 0: xv is input j of (state, own row); place j - 1 has been read
        }
        sy[c - c0] = acc / (1.0f + expf(-acc));
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float* orow = out + (size_t)row * channels;
    const int unit_end = unit_heads * unit_dim;
    if (c0 < unit_end) {
        const int h0 = c0 / unit_dim, h1 = min(unit_heads, (c1 + unit_dim - 1) / unit_dim);
        for (int head = h0 + warp; head < h1; head += nwarps) {
            const float* y = sy + (head * unit_dim - c0);
            float ss = 0.f;
            for (int d = lane; d < unit_dim; d += 32) ss += y[d] * y[d];
            ss = tw_warp_sum(ss);
            const float f = (head < scaled_heads ? head_scale : 1.0f) / sqrtf(ss + unit_eps);
            for (int d = lane; d < unit_dim; d += 32) orow[head * unit_dim + d] = y[d] * f;
        }
    }
    for (int c = max(c0, unit_end) + threadIdx.x; c < c1; c += blockDim.x) orow[c] = sy[c - c0];
}

// The same for steps with many rows and at most TW_CONV_FAST_TAPS taps: a block serves `rows_per_block` consecutive rows
// of the step, a thread keeps the last inputs of its channel in registers while it walks down the rows (an input is
// loaded once, not once per tap; the taps' weights once per block), and one barrier serves all the rows.  The taps
// are added in the same order as above, so both kernels give the same bits.
#define TW_CONV_FAST_TAPS 4
#define TW_CONV_ROWS 8
template <typename T, int TAPS>
__global__ void __launch_bounds__(256)
short_conv_rows_kernel(float* __restrict__ out, const T* __restrict__ x, int x_stride, const float* __restrict__ w,
                       float* __restrict__ state, long long state_stride, long long state_offset,
                       const int* __restrict__ seq_of_token, const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                       const int* __restrict__ seq_q_len, int move_single, int n_rows, int channels, int chunk, int unit_heads,
                       int unit_dim, int scaled_heads, float head_scale, float unit_eps) {
    extern __shared__ float sy[];        // [TW_CONV_ROWS][chunk]
    constexpr int R = TW_CONV_ROWS;
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int row0 = blockIdx.x * R;
    const int nr = min(R, n_rows - row0);
    const int c0 = blockIdx.y * chunk, c1 = min(channels, c0 + chunk);
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float wt[TAPS], xw[TAPS];
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wt[j] = w[(size_t)c * TAPS + j];
        // xw[j] is the input TAPS - 1 - j rows before the current one (whichever request that row belongs to)
#pragma unroll
        for (int j = 0; j + 1 < TAPS; ++j) {
            const int rr = row0 - (TAPS - 1) + j;
            xw[j] = rr >= 0 ? tw_to_float(x[(size_t)rr * x_stride + c]) : 0.f;
        }
        float xr[R];                     // the block's rows of this channel, all asked for before the first is used
#pragma unroll
        for (int i = 0; i < R; ++i) xr[i] = i < nr ? tw_to_float(x[(size_t)(row0 + i) * x_stride + c]) : 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            if (i >= nr) break;
            const int row = row0 + i;
            xw[TAPS - 1] = xr[i];
            const int s = seq_of_token[row];
            if (s >= 0) {
                const int r = row - seq_q_start[s];          // rows of this request before this one in the step
                float* tc = state + (size_t)seq_slot[s] * state_stride + state_offset + (size_t)c * (TAPS - 1);
                const bool move = move_single && TAPS > 1 && seq_q_len[s] == 1;
                float acc = 0.f;
#pragma unroll
                for (int j = 0; j < TAPS; ++j) {
                    const int back = TAPS - 1 - j;
                    const float xv = back <= r ? xw[j] : tc[TAPS - 1 + r - back];
                    acc += wt[j] * xv;
                    if (move && j > 0) tc[j - 1] = xv;
                }
                sy[i * chunk + (c - c0)] = acc / (1.0f + expf(-acc));
            }
#pragma unroll
            for (int j = 0; j + 1 < TAPS; ++j) xw[j] = xw[j + 1];
        }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int unit_end = unit_heads * unit_dim;
    const int h0 = unit_dim > 0 ? c0 / unit_dim : 0;
    const int h1 = c0 < unit_end ? min(unit_heads, (c1 + unit_dim - 1) / unit_dim) : h0;
    const int nh = h1 - h0;
    for (int pair = warp; pair < nr * nh; pair += nwarps) {
        const int i = pair / nh, head = h0 + (pair - i * nh);
        if (seq_of_token[row0 + i] < 0) continue;
        const float* y = sy + i * chunk + (head * unit_dim - c0);
        float ss = 0.f;
        for (int d = lane; d < unit_dim; d += 32) ss += y[d] * y[d];
        ss = tw_warp_sum(ss);
        const float f = (head < scaled_heads ? head_scale : 1.0f) / sqrtf(ss + unit_eps);
        float* orow = out + (size_t)(row0 + i) * channels;
        for (int d = lane; d < unit_dim; d += 32) orow[head * unit_dim + d] = y[d] * f;
    }
    const int p0 = max(c0, unit_end);
    if (p0 < c1) {
        const int span = c1 - p0;
        for (int e = threadIdx.x; e < nr * span; e += blockDim.x) {
            const int i = e / span, c = p0 + (e - i * span);
            if (seq_of_token[row0 + i] >= 0) out[(size_t)(row0 + i) * channels + c] = sy[i * chunk + (c - c0)];
        }
    }
}

// The convolution's state after the step: the last taps - 1 inputs of every request, older ones kept where the
// step brought fewer rows than that.  One thread per (request, channel) reads its old values before it writes.
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ x, int x_stride, int taps, float* __restrict__ state,
                                        long long state_stride, long long state_offset, const int* __restrict__ seq_slot,
                                        const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len, int channels,
                                        int skip_single) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int len = seq_q_len[s];
    if (c >= channels || len <= 0 || (skip_single && len == 1)) return;     // (tw_short_conv has moved the single rows' state on)
    const int start = seq_q_start[s], keep = taps - 1;
    float* tail = state + (size_t)seq_slot[s] * state_stride + state_offset + (size_t)c * keep;
    float fresh[16];
    for (int j = 0; j < keep; ++j) {
        const int r = len - keep + j;                    // the step's row that lands at place j (negative: an older one)
        fresh[j] = r >= 0 ? tw_to_float(x[(size_t)(start + r) * x_stride + c]) : tail[j + len];
    }
    for (int j = 0; j < keep; ++j) tail[j] = fresh[j];
}

template <typename T>
static int launch_short_conv(float* out, const T* x, int x_stride, const float* w, int taps, float* state, long long state_stride,
                             long long state_offset, const int* seq_of_token, const int* seq_slot, const int* seq_q_start,
                             const int* seq_q_len, int move_single, int n_rows, int channels, int unit_heads, int unit_dim,
                             int scaled_heads, float head_scale, float unit_eps, cudaStream_t stream) {
    // about 512 channels per block, in whole unit heads while there are any (a head larger than that has a block of its own)
    int chunk = 512;
    if (unit_heads > 0 && unit_dim > 0) chunk = unit_dim * (unit_dim >= 512 ? 1 : 512 / unit_dim);
    const size_t smem = (size_t)chunk * sizeof(float);
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(short_conv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (n_rows >= 8 * TW_CONV_ROWS && taps <= TW_CONV_FAST_TAPS && smem * TW_CONV_ROWS <= 96 * 1024) {
        const size_t rsmem = smem * TW_CONV_ROWS;
        const dim3 rgrid((n_rows + TW_CONV_ROWS - 1) / TW_CONV_ROWS, (channels + chunk - 1) / chunk);
#define TW_CONV_ROWS_LAUNCH(TAPS)                                                                                                \
        {                                                                                                                        \
            if (rsmem > 48 * 1024) {                                                                                             \
                const cudaError_t e = cudaFuncSetAttribute(short_conv_rows_kernel<T, TAPS>,                                      \
                                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rsmem);             \
                if (e != cudaSuccess) return (int)e;                                                                             \
            }                                                                                                                    \
            return tw_launch(short_conv_rows_kernel<T, TAPS>, rgrid, dim3(256), rsmem, stream, 1, out, x, x_stride, w, state,    \
                             state_stride, state_offset, seq_of_token, seq_slot, seq_q_start, seq_q_len, move_single, n_rows,   \
                             channels, chunk, unit_heads, unit_dim, scaled_heads, head_scale, unit_eps);                         \
        }
        switch (taps) {
        case 1: TW_CONV_ROWS_LAUNCH(1)
        case 2: TW_CONV_ROWS_LAUNCH(2)
        case 3: TW_CONV_ROWS_LAUNCH(3)
        default: TW_CONV_ROWS_LAUNCH(4)
        }
#undef TW_CONV_ROWS_LAUNCH
    }
    const dim3 grid(n_rows, (channels + chunk - 1) / chunk);
    return tw_launch(short_conv_kernel<T>, grid, dim3(256), smem, stream, 1, out, x, x_stride, w, taps, state, state_stride,
                     state_offset, seq_of_token, seq_slot, seq_q_start, seq_q_len, move_single, channels, chunk, unit_heads,
                     unit_dim, scaled_heads, head_scale, unit_eps);
}

// seq_q_len with move_single: requests that bring one row have their state moved on by this kernel (and
// tw_short_conv_state is then told to skip them).
TW_EXPORT int tw_short_conv(float* out, const void* x, int x_stride, const float* w, int taps, float* state,
                            long long state_stride, long long state_offset, const int* seq_of_token, const int* seq_slot,
                            const int* seq_q_start, const int* seq_q_len, int move_single, int n_rows, int channels,
                            int unit_heads, int unit_dim, int scaled_heads, float head_scale, float unit_eps, int dtype,
                            cudaStream_t stream) {
    if (n_rows <= 0 || channels <= 0) return 0;
    if (taps < 1 || taps > 17 || unit_heads * unit_dim > channels || (move_single && !seq_q_len)) return (int)cudaErrorInvalidValue;
    if (dtype == TW_F32)
        return launch_short_conv<float>(out, (const float*)x, x_stride, w, taps, state, state_stride, state_offset, seq_of_token,
                                        seq_slot, seq_q_start, seq_q_len, move_single, n_rows, channels, unit_heads, unit_dim,
                                        scaled_heads, head_scale, unit_eps, stream);
    return launch_short_conv<__nv_bfloat16>(out, (const __nv_bfloat16*)x, x_stride, w, taps, state, state_stride, state_offset,
                                            seq_of_token, seq_slot, seq_q_start, seq_q_len, move_single, n_rows, channels,
                                            unit_heads, unit_dim, scaled_heads, head_scale, unit_eps, stream);
}

TW_EXPORT int tw_short_conv_state(const void* x, int x_stride, int taps, float* state, long long state_stride,
                                  long long state_offset, const int* seq_slot, const int* seq_q_start, const int* seq_q_len,
                                  int n_seqs, int channels, int skip_single, int dtype, cudaStream_t stream) {
    if (n_seqs <= 0 || channels <= 0 || taps <= 1) return 0;
    if (taps > 17) return (int)cudaErrorInvalidValue;
    const dim3 grid((channels + 127) / 128, n_seqs);
    if (dtype == TW_F32)
        return tw_launch(short_conv_state_kernel<float>, grid, dim3(128), 0, stream, 1, (const float*)x, x_stride, taps, state,
                         state_stride, state_offset, seq_slot, seq_q_start, seq_q_len, channels, skip_single);
    return tw_launch(short_conv_state_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, 1, (const __nv_bfloat16*)x, x_stride, taps,
                     state, state_stride, state_offset, seq_slot, seq_q_start, seq_q_len, channels, skip_single);
}
