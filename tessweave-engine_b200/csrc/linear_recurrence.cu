// Linear attention as a recurrence over a matrix state of fixed size per request and head.
//
// A head keeps S [Dk, Dv] in fp32.  Several update rules share one kernel (rows q/r, k [Dk], v [Dv] per token):
//
//   TW_REC_RETENTION   S <- g S + k v^T                     o = S^T q          g a constant per head
//                      q and k are rotated by position on the way in, k is scaled after the rotation
//   TW_REC_WKV         o = (S + diag(u) k v^T)^T r          S <- diag(w) S + k v^T
//                      w = exp(-exp(d + w0)) per key channel from the projected d; u a bonus for the token itself
//   TW_REC_MLSTM       m' = max(f + m, i)                   S <- e^(f + m - m') S + e^(i - m') k v^T
//                      n likewise with k alone;  o = S^T q,  den = max(|n . q|, e^(-m')) + 1e-6
//                      i = cap tanh((pi + bi) / cap), f = logsigmoid(cap tanh((pf + bf) / cap)); m is 0 before
//                      the first token.  n is carried as one more column of S (a value that is always 1).
//   TW_REC_DELTA       S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q      (the gated delta rule)
//                      g = exp(-exp(A_h) softplus(d + b)) per head, or per head and key channel, from the projected d;
//                      beta = sigmoid of a projected number per head.  q and k arrive as fp32 rows that the caller has
//                      prepared (here: convolved, activated, scaled to unit length); heads of v may share a head of q
//                      and k (qk_group value heads per q/k head).  The read-out sees the token's own write:
//                      o = (gS)^T q + u (k . q), so one pass over the column gives (gS)^T k, (gS)^T q and k . q.
//   TW_REC_GLA         S <- diag(a) S + k v^T                o = S^T q          (gated linear attention)
//                      a = sigmoid(z + b)^(1 / tau) per key channel from the projected z, evaluated as
//                      exp(logsigmoid(z + b) / tau); 1 / tau arrives in `cap`, b in p0
//
// One block per (head, request, slice of the columns of S): a thread owns a column of S in registers (TW_DK
// values, a compile-time size; where that size is a multiple of 16 four or eight lanes share a column, a quarter or
// an eighth of its key channels each) and walks the request's rows of this step in order (the columns of a head are
// independent of one another, so a head is spread over as many blocks as it takes to fill the GPU; in steps with
// long portions the block's other warps stage the next 16 tokens meanwhile); the rows of 16 tokens at a time are staged in
// shared memory as fp32 (rotation, scaling, decays and gates are evaluated there, once per value).  The
// state slot is read at the first row and written back after the last, so a request may be cut into
// steps anywhere, and the sums at a position are formed in the same order however it was cut.  Outputs are
// fp32; the norm over a head, the gate and the rounding follow in tw_head_norm_gate (recurrent.cu).
#include "common.cuh"

#ifndef TW_DK
#define TW_DK 64
#endif
#define TW_REC_CHUNK 16
// A column's sums over the key channels are formed in TW_REC_SHARES shares of consecutive channels (four partial sums
// per share over the channels i mod 4, then the shares pairwise: neighbours, then neighbouring pairs, ...).  KS threads
// share a column, each with TW_REC_SHARES / KS of the shares (a warp serves 32 / KS columns; lanes l, l + that many, ...
// share one) and add across threads by shuffles in the same pairing: steps with long portions run KS = 8 where the key
// size allows (half the chain per token), steps of single tokens KS = 4 (wider reads of the state), and both give the
// same bits.
#define TW_REC_SHARES ((TW_DK % 32 == 0) ? 8 : ((TW_DK % 16 == 0) ? 4 : 1))

enum : int { TW_REC_RETENTION = 0, TW_REC_WKV = 1, TW_REC_MLSTM = 2, TW_REC_DELTA = 3, TW_REC_GLA = 4 };

struct RecArgs {
    float* out;                 // [rows, H * Dv] fp32
    float* den;                 // [rows, H] fp32 (mlstm)
    const void* q; int q_stride;        // rows of q (r), k, v: element type T, column h * D + i inside each
    const void* k; int k_stride;
    const void* v; int v_stride;
    const float* wpre; int wpre_stride; // wkv, gla: d [rows, H * Dk] fp32;  mlstm: [rows, 2 H] fp32 (pi | pf);  delta: d [rows, H * Dk] or [rows, H]
    const float* p0;            // wkv: w0 [H * Dk];  gla: b [H * Dk];  retention: decay [H];  mlstm: bias [2 H];  delta: A [H] (log of the rate)
    const float* p1;            // wkv: u [H * Dk];  delta: b [H * Dk] or [H]
    const float* bpre; int bpre_stride; // delta: the write strength's pre-activation [rows, H] fp32
    int channel_decay;          // delta: a decay per key channel (else one per head)
    int qk_group;               // value heads that share a head of q and k (1: every head has its own)
    const float* inv_freq; int rot_dims;    // retention: rotation of the first rot_dims values of q and k
    float k_scale, q_scale, cap;
    float* state; long long state_stride;  // [slots, state_stride]; a head's part starts at h * head_state
    const void* tail_src; int tail_stride, tail_width; long long tail_offset;   // wkv: row copied behind the heads
    const int* positions;
    const int* seq_slot; const int* seq_q_start; const int* seq_q_len;
    int H, Dv, write_state;
    int cols_per_block;         // columns of S a block owns (its first `cols_per_block` threads; all threads stage rows)
};

__device__ __forceinline__ float tw_logsigmoid(float x) {
    return fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
}
__device__ __forceinline__ float tw_softplus(float x) {
    return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
}

template <typename T, int MODE, int KS>
__global__ void __launch_bounds__(512)
linear_recurrence_kernel(RecArgs a) {
    extern __shared__ float sm[];
    constexpr int DK = TW_DK, C = TW_REC_CHUNK, SK = DK / KS;
    constexpr int NSH = KS > 1 ? TW_REC_SHARES / KS : 1, SH = SK / NSH;    // shares per thread, channels per share
    // A staged row keeps the KS shares of its key channels four floats apart (SEG = SK + 4), so that the four 16-byte
    // reads a warp issues at once (one per share) fall into different banks; DKP is the padded row.
    constexpr int SEG = SK + (KS > 1 ? 4 : 0), DKP = SEG * KS;
    auto pad = [](int i) { return KS > 1 ? i + 4 * (i / SK) : i; };
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int h = blockIdx.x, s = blockIdx.y;
    const int len = a.seq_q_len[s];
    if (len <= 0) return;
    const int start = a.seq_q_start[s];
    const int Dv = a.Dv, cols = MODE == TW_REC_MLSTM ? Dv + 1 : Dv;
    const int per = a.cols_per_block;
    // the block's first per * KS threads walk the state: with KS > 1 a warp serves CPW = 32 / KS columns (lane % CPW) and
    // a lane the key channels [ks * SK, (ks + 1) * SK) with ks = lane / CPW; with KS = 1 a thread serves a whole column
    constexpr int CPW = 32 / KS;
    const int jl = KS == 1 ? (int)threadIdx.x : (int)(threadIdx.x >> 5) * CPW + (int)(threadIdx.x & (CPW - 1));
    const int ks = KS == 1 ? 0 : (int)(threadIdx.x & 31) / CPW;
    const int j = blockIdx.z * per + jl;
    const bool walks = (int)threadIdx.x < per * KS;  // the threads that own (a share of) a column; the others only stage rows
    const bool live = walks && j < cols;
    // a staged chunk: q [C][DK], k [C][DK], w [C][DK] (wkv) or gates [C][2] (mlstm), v [C][per]; two of them, so that
    // the rows of the next 16 tokens are staged while the state walks through these
    const int extra = (MODE == TW_REC_WKV || MODE == TW_REC_GLA) ? C * DKP : (MODE == TW_REC_MLSTM ? 2 * C : (MODE == TW_REC_DELTA ? C * DKP + 2 * C : 0));
    const int chunk_floats = 2 * C * DKP + extra + C * per;
    float* su = sm + 2 * chunk_floats;      // [DKP] bonus (wkv)
    const long long head_state = (long long)DK * cols + (MODE == TW_REC_MLSTM ? 1 : 0);
    float* slot = a.state + (size_t)a.seq_slot[s] * a.state_stride + (size_t)h * head_state;
    const T* __restrict__ gq = (const T*)a.q;
    const T* __restrict__ gk = (const T*)a.k;
    const T* __restrict__ gv = (const T*)a.v;
    const int half = a.rot_dims >> 1;
    const int hq = h / a.qk_group;      // the head of q and k this head reads
    const float rate = MODE == TW_REC_DELTA ? expf(a.p0[h]) : 0.f;     // delta: the head's decay rate
    const bool vec_rows = MODE == TW_REC_DELTA && sizeof(T) == 4 && (a.q_stride % 4) == 0 && (a.k_stride % 4) == 0
                          && (reinterpret_cast<size_t>(a.q) % 16) == 0 && (reinterpret_cast<size_t>(a.k) % 16) == 0
                          && (!a.channel_decay || ((a.wpre_stride % 4) == 0 && (reinterpret_cast<size_t>(a.wpre) % 16) == 0
                                                   && (reinterpret_cast<size_t>(a.p1) % 16) == 0));

    const bool vec_gla = MODE == TW_REC_GLA && sizeof(T) == 2 && (a.q_stride % 8) == 0 && (a.k_stride % 8) == 0
                         && (reinterpret_cast<size_t>(a.q) % 16) == 0 && (reinterpret_cast<size_t>(a.k) % 16) == 0
                         && (a.wpre_stride % 4) == 0 && (reinterpret_cast<size_t>(a.wpre) % 16) == 0
                         && (reinterpret_cast<size_t>(a.p0) % 16) == 0;

    // ---- the rows of up to C tokens from t0 on, as fp32: rotation, scaling, decays and gates are evaluated here
    auto stage = [&](int t0, float* buf, int tid, int nthreads) {
        const int ct = min(C, len - t0);
        float* sq = buf;
        float* sk = sq + C * DKP;
        float* sw = sk + C * DKP;
        float* sv = sw + extra;
        if (MODE == TW_REC_RETENTION) {
            // a rotated pair (i, i + half) at a time: one angle, four loads, four values
            for (int e = tid; e < ct * half; e += nthreads) {
                const int t = e / half, i = e - t * half;
                const size_t row = (size_t)(start + t0 + t);
                const T* qr = gq + row * a.q_stride + hq * DK;
                const T* kr = gk + row * a.k_stride + hq * DK;
                const float q1 = tw_to_float(qr[i]), q2 = tw_to_float(qr[i + half]);
                const float k1 = tw_to_float(kr[i]), k2 = tw_to_float(kr[i + half]);
                float sn, cs;
                sincosf((float)a.positions[row] * a.inv_freq[i], &sn, &cs);
                sq[t * DKP + pad(i)] = (q1 * cs - q2 * sn) * a.q_scale;
                sq[t * DKP + pad(i + half)] = (q2 * cs + q1 * sn) * a.q_scale;
                sk[t * DKP + pad(i)] = (k1 * cs - k2 * sn) * a.k_scale;
                sk[t * DKP + pad(i + half)] = (k2 * cs + k1 * sn) * a.k_scale;
            }
        }
        const int first = MODE == TW_REC_RETENTION ? a.rot_dims : 0;     // channels from here on are not rotated
        const int plain = DK - first;
        bool staged = false;
        if constexpr (MODE == TW_REC_DELTA && sizeof(T) == 4 && KS > 1) {
            if (vec_rows) {
                // fp32 rows whose heads start on 16-byte boundaries: four channels per load, and all of a thread's
                // loads of the chunk are under way before the first is used
                constexpr int V = DK / 4;
#pragma unroll 2
                for (int e = tid; e < ct * V; e += nthreads) {
                    const int t = e / V, i = 4 * (e - t * V);
                    const size_t row = (size_t)(start + t0 + t);
                    float4 qq = *reinterpret_cast<const float4*>((const float*)gq + row * a.q_stride + hq * DK + i);
                    float4 kk = *reinterpret_cast<const float4*>((const float*)gk + row * a.k_stride + hq * DK + i);
                    qq.x *= a.q_scale; qq.y *= a.q_scale; qq.z *= a.q_scale; qq.w *= a.q_scale;
                    kk.x *= a.k_scale; kk.y *= a.k_scale; kk.z *= a.k_scale; kk.w *= a.k_scale;
                    if (a.channel_decay) {
                        const float4 dd = *reinterpret_cast<const float4*>(a.wpre + row * a.wpre_stride + h * DK + i);
                        const float4 bb = *reinterpret_cast<const float4*>(a.p1 + h * DK + i);
                        float4 ww;
                        ww.x = expf(-rate * tw_softplus(dd.x + bb.x));
                        ww.y = expf(-rate * tw_softplus(dd.y + bb.y));
                        ww.z = expf(-rate * tw_softplus(dd.z + bb.z));
                        ww.w = expf(-rate * tw_softplus(dd.w + bb.w));
                        *reinterpret_cast<float4*>(sw + t * DKP + pad(i)) = ww;
                    }
                    *reinterpret_cast<float4*>(sq + t * DKP + pad(i)) = qq;
                    *reinterpret_cast<float4*>(sk + t * DKP + pad(i)) = kk;
                }
                staged = true;
            }
        }
        if constexpr (MODE == TW_REC_GLA && sizeof(T) == 2 && KS > 1 && DK % 8 == 0) {
            if (vec_gla) {
                // (the same arithmetic as one channel at a time.  The wkv rule's rows were staged this way too, and its
                // 56 heads of 64 gained nothing: 528 us against 533 for 2,048 tokens; it keeps the loop below)
                auto decay_of = [&](float x) { return expf(tw_logsigmoid(x) * a.cap); };
                // bf16 rows whose heads start on 16-byte boundaries: four channels per load (8 bytes of q and of k, 16 of the
                // projected decay and of its bias), and eight channels per thread and step where a head is wide enough to keep
                // every staging thread busy that way; all of a thread's loads are under way before the first is used
                constexpr int W = DK >= 128 ? 8 : 4, V = DK / W;
                for (int e = tid; e < ct * V; e += nthreads) {
                    const int t = e / V, i0 = W * (e - t * V);
                    const size_t row = (size_t)(start + t0 + t);
                    uint2 qraw[W / 4], kraw[W / 4];
                    float4 dd[W / 4], bb[W / 4];
#pragma unroll
                    for (int g = 0; g < W / 4; ++g) {
                        const int i = i0 + 4 * g;
                        qraw[g] = *reinterpret_cast<const uint2*>(gq + row * a.q_stride + hq * DK + i);
                        kraw[g] = *reinterpret_cast<const uint2*>(gk + row * a.k_stride + hq * DK + i);
                        dd[g] = *reinterpret_cast<const float4*>(a.wpre + row * a.wpre_stride + h * DK + i);
                        bb[g] = *reinterpret_cast<const float4*>(a.p0 + h * DK + i);
                    }
                    const float qs = a.q_scale, ks_ = a.k_scale;
#pragma unroll
                    for (int g = 0; g < W / 4; ++g) {
                        const int i = i0 + 4 * g;
                        const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&qraw[g]);
                        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kraw[g]);
                        const float2 qa = __bfloat1622float2(q2[0]), qb = __bfloat1622float2(q2[1]);
                        const float2 ka = __bfloat1622float2(k2[0]), kb = __bfloat1622float2(k2[1]);
                        *reinterpret_cast<float4*>(sq + t * DKP + pad(i)) = make_float4(qa.x * qs, qa.y * qs, qb.x * qs, qb.y * qs);
                        *reinterpret_cast<float4*>(sk + t * DKP + pad(i)) = make_float4(ka.x * ks_, ka.y * ks_, kb.x * ks_, kb.y * ks_);
                        *reinterpret_cast<float4*>(sw + t * DKP + pad(i)) =
                            make_float4(decay_of(dd[g].x + bb[g].x), decay_of(dd[g].y + bb[g].y), decay_of(dd[g].z + bb[g].z),
                                        decay_of(dd[g].w + bb[g].w));
                    }
                }
                staged = true;
            }
        }
        if (!staged) {
#pragma unroll 4
            for (int e = tid; e < ct * plain; e += nthreads) {
                const int t = e / plain, i = first + (e - t * plain);
                const size_t row = (size_t)(start + t0 + t);
                sq[t * DKP + pad(i)] = tw_to_float(gq[row * a.q_stride + hq * DK + i]) * a.q_scale;
                sk[t * DKP + pad(i)] = tw_to_float(gk[row * a.k_stride + hq * DK + i]) * a.k_scale;
                if (MODE == TW_REC_WKV)
                    sw[t * DKP + pad(i)] = expf(-expf(a.wpre[row * a.wpre_stride + h * DK + i] + a.p0[h * DK + i]));
                if (MODE == TW_REC_GLA)
                    sw[t * DKP + pad(i)] = expf(tw_logsigmoid(a.wpre[row * a.wpre_stride + h * DK + i] + a.p0[h * DK + i]) * a.cap);
                if (MODE == TW_REC_DELTA && a.channel_decay)
                    sw[t * DKP + pad(i)] = expf(-rate * tw_softplus(a.wpre[row * a.wpre_stride + h * DK + i] + a.p1[h * DK + i]));
            }
        }
        if (MODE == TW_REC_DELTA) {
            float* sg = sw + C * DKP;       // [C] the head's decay (where it has one for all channels), [C] the write strength
            for (int t = tid; t < ct; t += nthreads) {
                const size_t row = (size_t)(start + t0 + t);
                if (!a.channel_decay) sg[t] = expf(-rate * tw_softplus(a.wpre[row * a.wpre_stride + h] + a.p1[h]));
                sg[C + t] = 1.0f / (1.0f + expf(-a.bpre[row * a.bpre_stride + h]));
            }
        }
        for (int e = tid; e < ct * per; e += nthreads) {     // the block's own columns of v
            const int t = e / per, c = blockIdx.z * per + (e - t * per);
            if (c < Dv) sv[e] = tw_to_float(gv[(size_t)(start + t0 + t) * a.v_stride + h * Dv + c]);
        }
        if (MODE == TW_REC_MLSTM) {
            for (int t = tid; t < ct; t += nthreads) {
                const float* g = a.wpre + (size_t)(start + t0 + t) * a.wpre_stride;
                const float pi = g[h] + a.p0[h], pf = g[a.H + h] + a.p0[a.H + h];
                sw[2 * t] = a.cap * tanhf(pi / a.cap);
                sw[2 * t + 1] = tw_logsigmoid(a.cap * tanhf(pf / a.cap));
            }
        }
    };

    float S[SK];
    float m = 0.f;
    if (live) {
#pragma unroll
        for (int i = 0; i < SK; ++i) S[i] = slot[(size_t)(ks * SK + i) * cols + j];
    }
    if (MODE == TW_REC_MLSTM) m = slot[(size_t)DK * cols];
    if (MODE == TW_REC_WKV) {
        for (int i = threadIdx.x; i < DK; i += blockDim.x) su[pad(i)] = a.p1[h * DK + i];
    }
    const float decay = MODE == TW_REC_RETENTION ? a.p0[h] : 0.f;
    const int stagers = (int)blockDim.x - per * KS;  // threads that own no column

    stage(0, sm, threadIdx.x, blockDim.x);
    __syncthreads();
    for (int t0 = 0, c = 0; t0 < len; t0 += C, ++c) {
        const int ct = min(C, len - t0);
        float* buf = sm + (c & 1) * chunk_floats;
        float* next = sm + ((c + 1) & 1) * chunk_floats;
        const bool more = t0 + C < len;
        if (!walks && more) stage(t0 + C, next, threadIdx.x - per * KS, stagers);
        if (walks) {                                 // (threads of a live warp whose column lies beyond the last take part in its shuffles)
            const float* sq = buf;
            const float* sk = sq + C * DKP;
            const float* sw = sk + C * DKP;
            const float* sv = sw + extra;
            // ---- the recurrence, token by token
            for (int t = 0; t < ct; ++t) {
                const float* q = sq + t * DKP + ks * SEG;
                const float* k = sk + t * DKP + ks * SEG;
                const float vj = (MODE == TW_REC_MLSTM && j == Dv) ? 1.f : (j < Dv ? sv[t * per + jl] : 0.f);
                // four partial sums (key channels i mod 4), added at the end: the same order in every step, whatever its size
                float acc4[4] = {0.f, 0.f, 0.f, 0.f};
                float fa = 0.f, fb = 0.f;
                if (MODE == TW_REC_MLSTM) {
                    const float li = sw[2 * t], lf = sw[2 * t + 1];
                    const float m_new = fmaxf(lf + m, li);
                    fa = expf(lf + m - m_new);
                    fb = expf(li - m_new) * vj;
                    m = m_new;
                }
                const float* w = sw + t * DKP + ks * SEG;
                const float* u = su + ks * SEG;
                if constexpr (MODE == TW_REC_DELTA) {
                    // one pass: decay the column, and form its products with k and with q, and k . q (four partial sums
                    // each over the key channels i mod 4, the same order in every step)
                    const float gh = a.channel_decay ? 1.f : sw[C * DKP + t];
                    const float beta = sw[C * DKP + C + t];
                    float r4[4] = {0.f, 0.f, 0.f, 0.f}, d4[4] = {0.f, 0.f, 0.f, 0.f};
                    float rs[NSH], ps[NSH], ds[NSH];
                    if constexpr (SH % 4 == 0) {     // 16-byte reads of the staged rows; share by share
                        const float4* q4 = reinterpret_cast<const float4*>(q);
                        const float4* k4 = reinterpret_cast<const float4*>(k);
                        const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
                        for (int sh = 0; sh < NSH; ++sh) {
                            float rr[4] = {0.f, 0.f, 0.f, 0.f}, pp[4] = {0.f, 0.f, 0.f, 0.f}, dd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                            for (int i4 = sh * (SH / 4); i4 < (sh + 1) * (SH / 4); ++i4) {
                                const float4 qq = q4[i4], kk = k4[i4];
                                const float qa[4] = {qq.x, qq.y, qq.z, qq.w}, ka[4] = {kk.x, kk.y, kk.z, kk.w};
                                float ga[4] = {gh, gh, gh, gh};
                                if (a.channel_decay) {
                                    const float4 ww = w4[i4];
                                    ga[0] = ww.x; ga[1] = ww.y; ga[2] = ww.z; ga[3] = ww.w;
                                }
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int i = 4 * i4 + e;
                                    S[i] *= ga[e];
                                    rr[e] += S[i] * ka[e];
                                    pp[e] += S[i] * qa[e];
                                    dd[e] += ka[e] * qa[e];
                                }
                            }
                            rs[sh] = (rr[0] + rr[1]) + (rr[2] + rr[3]);
                            ps[sh] = (pp[0] + pp[1]) + (pp[2] + pp[3]);
                            ds[sh] = (dd[0] + dd[1]) + (dd[2] + dd[3]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < SK; ++i) {
                            const float g = a.channel_decay ? w[i] : gh;
                            S[i] *= g;
                            r4[i & 3] += S[i] * k[i];
                            acc4[i & 3] += S[i] * q[i];
                            d4[i & 3] += k[i] * q[i];
                        }
                    }
                    float r = (r4[0] + r4[1]) + (r4[2] + r4[3]);
                    float p = (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);
                    float d = (d4[0] + d4[1]) + (d4[2] + d4[3]);
                    if constexpr (SH % 4 == 0) {
                        static_assert(NSH == 1 || NSH == 2, "a thread holds one share or two neighbours");
                        r = NSH == 2 ? rs[0] + rs[NSH - 1] : rs[0];
                        p = NSH == 2 ? ps[0] + ps[NSH - 1] : ps[0];
                        d = NSH == 2 ? ds[0] + ds[NSH - 1] : ds[0];
                    }
                    if (KS > 1) {
#pragma unroll
                        for (int o = CPW; o < 32; o <<= 1) {
                            r += __shfl_xor_sync(0xffffffffu, r, o);
                            p += __shfl_xor_sync(0xffffffffu, p, o);
                            d += __shfl_xor_sync(0xffffffffu, d, o);
                        }
                    }
                    const float uj = beta * (vj - r);
                    if constexpr (SK % 4 == 0) {
                        const float4* k4 = reinterpret_cast<const float4*>(k);
#pragma unroll
                        for (int i4 = 0; i4 < SK / 4; ++i4) {
                            const float4 kk = k4[i4];
                            S[4 * i4] += kk.x * uj; S[4 * i4 + 1] += kk.y * uj;
                            S[4 * i4 + 2] += kk.z * uj; S[4 * i4 + 3] += kk.w * uj;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < SK; ++i) S[i] += k[i] * uj;
                    }
                    if (live && ks == 0)
                        a.out[(size_t)(start + t0 + t) * ((size_t)a.H * Dv) + (size_t)h * Dv + j] = p + uj * d;
                    continue;
                }
                float share_sum[NSH];
                if constexpr (SH % 4 == 0) {
                    const float4* q4 = reinterpret_cast<const float4*>(q);
                    const float4* k4 = reinterpret_cast<const float4*>(k);
                    const float4* w4 = reinterpret_cast<const float4*>(w);
                    const float4* u4 = reinterpret_cast<const float4*>(u);
#pragma unroll
                    for (int sh = 0; sh < NSH; ++sh) {
                    acc4[0] = acc4[1] = acc4[2] = acc4[3] = 0.f;
#pragma unroll
                    for (int i4 = sh * (SH / 4); i4 < (sh + 1) * (SH / 4); ++i4) {
                        const float4 qq = q4[i4], kk = k4[i4];
                        const float qa[4] = {qq.x, qq.y, qq.z, qq.w}, ka[4] = {kk.x, kk.y, kk.z, kk.w};
                        float wa[4] = {0.f, 0.f, 0.f, 0.f}, ua[4] = {0.f, 0.f, 0.f, 0.f};
                        if (MODE == TW_REC_WKV) {
                            const float4 ww = w4[i4], uu = u4[i4];
                            wa[0] = ww.x; wa[1] = ww.y; wa[2] = ww.z; wa[3] = ww.w;
                            ua[0] = uu.x; ua[1] = uu.y; ua[2] = uu.z; ua[3] = uu.w;
                        }
                        if (MODE == TW_REC_GLA) {
                            const float4 ww = w4[i4];
                            wa[0] = ww.x; wa[1] = ww.y; wa[2] = ww.z; wa[3] = ww.w;
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int i = 4 * i4 + e;
                            if (MODE == TW_REC_RETENTION) {
                                S[i] = decay * S[i] + ka[e] * vj;
                                acc4[e] += qa[e] * S[i];
                            } else if (MODE == TW_REC_WKV) {
                                const float kv = ka[e] * vj;
                                acc4[e] += qa[e] * (S[i] + ua[e] * kv);
                                S[i] = wa[e] * S[i] + kv;
                            } else if (MODE == TW_REC_GLA) {
                                S[i] = wa[e] * S[i] + ka[e] * vj;
                                acc4[e] += qa[e] * S[i];
                            } else {
                                S[i] = fa * S[i] + fb * ka[e];
                                acc4[e] += qa[e] * S[i];
                            }
                        }
                    }
                    share_sum[sh] = (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < SK; ++i) {
                        if (MODE == TW_REC_RETENTION) {
                            S[i] = decay * S[i] + k[i] * vj;
                            acc4[i & 3] += q[i] * S[i];
                        } else if (MODE == TW_REC_WKV) {
                            const float kv = k[i] * vj;
                            acc4[i & 3] += q[i] * (S[i] + u[i] * kv);
                            S[i] = w[i] * S[i] + kv;
                        } else if (MODE == TW_REC_GLA) {
                            S[i] = w[i] * S[i] + k[i] * vj;
                            acc4[i & 3] += q[i] * S[i];
                        } else {
                            S[i] = fa * S[i] + fb * k[i];
                            acc4[i & 3] += q[i] * S[i];
                        }
                    }
                }
                float acc = (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);
                if constexpr (SH % 4 == 0) acc = NSH == 2 ? share_sum[0] + share_sum[NSH - 1] : share_sum[0];
                if (KS > 1) {                        // the shares of a column, always added in this order
#pragma unroll
                    for (int o = CPW; o < 32; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                }
                const size_t row = (size_t)(start + t0 + t);
                if (live && ks == 0) {
                    if (MODE == TW_REC_MLSTM && j == Dv)
                        a.den[row * a.H + h] = fmaxf(fabsf(acc), expf(-m)) + 1e-6f;
                    else
                        a.out[row * ((size_t)a.H * Dv) + (size_t)h * Dv + j] = acc;
                }
            }
        }
        if (stagers <= 0 && more) {                  // every thread owns a column: they stage together, between the chunks
            __syncthreads();
            stage(t0 + C, next, threadIdx.x, blockDim.x);
        }
        __syncthreads();
    }
    if (!a.write_state) return;
    if (live) {
#pragma unroll
        for (int i = 0; i < SK; ++i) slot[(size_t)(ks * SK + i) * cols + j] = S[i];
    }
    if (MODE == TW_REC_MLSTM && live && j == 0 && ks == 0) slot[(size_t)DK * cols] = m;
    if (MODE == TW_REC_WKV && h == 0 && blockIdx.z == 0 && a.tail_src) {
        // what the next step's first token mixes with: the last row this mixer read
        const T* src = (const T*)a.tail_src + (size_t)(start + len - 1) * a.tail_stride;
        float* dst = a.state + (size_t)a.seq_slot[s] * a.state_stride + a.tail_offset;
        for (int c = threadIdx.x; c < a.tail_width; c += blockDim.x) dst[c] = tw_to_float(src[c]);
    }
}

template <typename T, int MODE, int KS>
static int launch_split(const RecArgs& a, int n_seqs, bool long_portions, cudaStream_t stream) {
    const int cols = MODE == TW_REC_MLSTM ? a.Dv + 1 : a.Dv;
    // columns per block: as many as still give the GPU a block per SM, at least a warp's worth.  A block has four
    // warps at least: all of them stage the rows (loads, rotation, decays), the first `per` threads walk the state
    constexpr int SEG = TW_DK / KS + (KS > 1 ? 4 : 0), DKP = SEG * KS;
    int per = KS == 1 ? 128 : 256 / KS;          // (per * KS walking threads and 256 that stage fit a block of 512)
    const int least = KS == 8 ? 16 : 32;
    while (per > least && (long long)a.H * n_seqs * ((cols + per - 1) / per) < 148) per >>= 1;
    if (per > ((cols + 31) / 32) * 32) per = ((cols + 31) / 32) * 32;
    RecArgs b = a;
    b.cols_per_block = per;
    const size_t chunk = 2 * TW_REC_CHUNK * DKP + (size_t)TW_REC_CHUNK * per
                         + ((MODE == TW_REC_WKV || MODE == TW_REC_GLA) ? TW_REC_CHUNK * DKP
                            : (MODE == TW_REC_MLSTM ? 2 * TW_REC_CHUNK : (MODE == TW_REC_DELTA ? TW_REC_CHUNK * DKP + 2 * TW_REC_CHUNK : 0)));
    const size_t smem = (2 * chunk + DKP) * sizeof(float);
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(linear_recurrence_kernel<T, MODE, KS>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    // steps of single tokens stage one chunk and walk it: a thread per column; longer portions get warps that only stage
    const int threads = long_portions ? per * KS + 256 : per * KS;
    return tw_launch(linear_recurrence_kernel<T, MODE, KS>, dim3(a.H, n_seqs, (cols + per - 1) / per), dim3(threads), smem, stream, 1, b);
}

template <typename T, int MODE>
static int launch_recurrence(const RecArgs& a, int n_seqs, bool long_portions, cudaStream_t stream) {
    if constexpr (TW_REC_SHARES == 8) {
        if (!long_portions) return launch_split<T, MODE, 4>(a, n_seqs, long_portions, stream);
    }
    return launch_split<T, MODE, TW_REC_SHARES>(a, n_seqs, long_portions, stream);
}

TW_EXPORT int tw_linear_recurrence(int mode, float* out, float* den, const void* q, int q_stride, const void* k, int k_stride,
                                   const void* v, int v_stride, const float* wpre, int wpre_stride, const float* p0,
                                   const float* p1, const float* bpre, int bpre_stride, int channel_decay, int qk_group,
                                   const float* inv_freq, int rot_dims, float q_scale, float k_scale,
                                   float cap, float* state, long long state_stride, const void* tail_src, int tail_stride,
                                   int tail_width, long long tail_offset, const int* positions, const int* seq_slot,
                                   const int* seq_q_start, const int* seq_q_len, int n_seqs, int H, int Dk, int Dv,
                                   int write_state, int max_q_len, int dtype, cudaStream_t stream) {
    if (n_seqs <= 0 || H <= 0) return 0;
    const bool lp = max_q_len > TW_REC_CHUNK;
    if (Dk != TW_DK || Dv <= 0 || Dv > 256 || rot_dims < 0 || rot_dims > Dk || (rot_dims & 1)) return (int)cudaErrorInvalidValue;
    if (qk_group <= 0 || H % qk_group) return (int)cudaErrorInvalidValue;
    RecArgs a;
    a.bpre = bpre; a.bpre_stride = bpre_stride; a.channel_decay = channel_decay; a.qk_group = qk_group;
    a.out = out; a.den = den; a.q = q; a.q_stride = q_stride; a.k = k; a.k_stride = k_stride; a.v = v; a.v_stride = v_stride;
    a.wpre = wpre; a.wpre_stride = wpre_stride; a.p0 = p0; a.p1 = p1; a.inv_freq = inv_freq; a.rot_dims = inv_freq ? rot_dims : 0;
    a.k_scale = k_scale; a.q_scale = q_scale; a.cap = cap; a.state = state; a.state_stride = state_stride;
    a.tail_src = tail_src; a.tail_stride = tail_stride; a.tail_width = tail_width; a.tail_offset = tail_offset;
    a.positions = positions; a.seq_slot = seq_slot; a.seq_q_start = seq_q_start; a.seq_q_len = seq_q_len;
    a.H = H; a.Dv = Dv; a.write_state = write_state; a.cols_per_block = 0;
    const bool f32 = dtype == TW_F32;
    switch (mode) {
    case TW_REC_RETENTION:
        return f32 ? launch_recurrence<float, TW_REC_RETENTION>(a, n_seqs, lp, stream)
                   : launch_recurrence<__nv_bfloat16, TW_REC_RETENTION>(a, n_seqs, lp, stream);
    case TW_REC_WKV:
        if (Dv != Dk) return (int)cudaErrorInvalidValue;
        return f32 ? launch_recurrence<float, TW_REC_WKV>(a, n_seqs, lp, stream)
                   : launch_recurrence<__nv_bfloat16, TW_REC_WKV>(a, n_seqs, lp, stream);
    case TW_REC_MLSTM:
        return f32 ? launch_recurrence<float, TW_REC_MLSTM>(a, n_seqs, lp, stream)
                   : launch_recurrence<__nv_bfloat16, TW_REC_MLSTM>(a, n_seqs, lp, stream);
    case TW_REC_GLA:
        if (!wpre || !p0) return (int)cudaErrorInvalidValue;
        return f32 ? launch_recurrence<float, TW_REC_GLA>(a, n_seqs, lp, stream)
                   : launch_recurrence<__nv_bfloat16, TW_REC_GLA>(a, n_seqs, lp, stream);
    case TW_REC_DELTA:
        if (!f32 || !bpre || !wpre || !p0 || !p1) return (int)cudaErrorInvalidValue;     // its rows are prepared in fp32 in every run type
        return launch_recurrence<float, TW_REC_DELTA>(a, n_seqs, lp, stream);
    }
    return (int)cudaErrorInvalidValue;
}
