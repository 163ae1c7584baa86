// Kernels of mixers and norms beyond the softmax-attention decoder: layer norm (on a sublayer's output, added into the
// stream; or of chosen rows), gated feed-forward activations, short causal convolutions over time with their per-request
// tails, whole-projection RMS norm and partial interleaved rotation of queries and keys, linear-attention recurrences
// with a constant or a projected decay, and the norm + gate that follows them.
//
// Everything a recurrence touches is float32: the state, the decays and their logarithms, the gates, the norms.  The
// projections arrive as float32 rows of one fused product ([q | k | v | gate | ...] side by side, `ld` apart); what the
// next product reads is written in the activation type T (float or bfloat16), rounded once.
//
// A step's rows are laid out request after request: request i owns rows req_start[i] .. req_start[i+1]-1, which continue
// the sequence at position req_pos[i]; its state lives in slot slot_ids[i] of each state tensor.  A kernel that carries
// state reads what earlier steps left and leaves what later steps need, so a whole prompt, a portion and a single token
// are one case.
#include "common.cuh"
#include "host_rules.h"

#include <algorithm>

JK_DEFINE_ERROR_BUFFER(jk_mixers)

// accurate forms: no fast-math anywhere in this package
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
// log(sigmoid(z)) without overflow on either side
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

enum MixAct : int { ACT_NONE = 0, ACT_SILU = 1, ACT_GELU_TANH = 2, ACT_SIGMOID = 3, ACT_RELU = 4, ACT_GELU_ERF = 5, ACT_TANH = 7 };
__device__ __forceinline__ float apply_act(int act, float z) {
    switch (act) {
        case ACT_SILU: return silu_f(z);
        case ACT_GELU_TANH: return gelu_tanh_f(z);
        case ACT_SIGMOID: return sigmoid_f(z);
        case ACT_RELU: return fmaxf(z, 0.f);
        case ACT_GELU_ERF: return 0.5f * z * (1.f + erff(z * 0.7071067811865476f));
        case ACT_TANH: return tanhf(z);
        default: return z;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Layer norm: y = (v - mean(v)) / sqrt(mean((v - mean)^2) + eps) * w + b, one block per row, the row held in shared
// memory between the passes (mean first, then the mean of the squared deviations).
//   add mode   (x_add != null): v = delta[r]; x[r] += y; h[r] = T(x[r]) if h is given      (norm on a sublayer's output)
//   rows mode  (x_add == null): v = x[rows ? rows[i] : i]; out[i] = T(y)                     (a norm that feeds a product)
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void store4_as(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store4_as(__nv_bfloat16 *p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned *>(&lo); raw.y = *reinterpret_cast<const unsigned *>(&hi);
    *reinterpret_cast<uint2 *>(p) = raw;
}

// VEC: the width is a multiple of 4 (rows of every operand then start on 16-byte boundaries: four elements move at a time)
template <typename T, bool VEC>
__global__ void layernorm_kernel(const float *__restrict__ src, const int *__restrict__ rows, const float *__restrict__ w,
                                 const float *__restrict__ b, float eps, float *__restrict__ x_add, T *__restrict__ out, int d) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    const float *v = src + (size_t)r * d;
    float s = 0.f;
    if (VEC) {
        for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
            const float4 t = *reinterpret_cast<const float4 *>(v + c);
            *reinterpret_cast<float4 *>(row_buf + c) = t;
            s += (t.x + t.y) + (t.z + t.w);
        }
    } else {
        for (int c = threadIdx.x; c < d; c += blockDim.x) {
            const float t = v[c];
            row_buf[c] = t;
            s += t;
        }
    }
    const float mean = block_sum(s, scratch) / (float)d;
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        const float t = row_buf[c] - mean;
        ss += t * t;
    }
    const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
    if (VEC) {
        for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
            const float4 t = *reinterpret_cast<const float4 *>(row_buf + c), ww = *reinterpret_cast<const float4 *>(w + c);
            const float4 bb = b ? *reinterpret_cast<const float4 *>(b + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 y = make_float4((t.x - mean) * inv * ww.x + bb.x, (t.y - mean) * inv * ww.y + bb.y,
                                   (t.z - mean) * inv * ww.z + bb.z, (t.w - mean) * inv * ww.w + bb.w);
            if (x_add != nullptr) {
                float *xp = x_add + (size_t)r * d + c;
                const float4 x = *reinterpret_cast<const float4 *>(xp);
                y = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
                *reinterpret_cast<float4 *>(xp) = y;
                if (out != nullptr) store4_as(out + (size_t)i * d + c, y);
            } else {
                store4_as(out + (size_t)i * d + c, y);
            }
        }
    } else {
        for (int c = threadIdx.x; c < d; c += blockDim.x) {
            const float y = (row_buf[c] - mean) * inv * w[c] + (b ? b[c] : 0.f);
            if (x_add != nullptr) {
                const float nx = x_add[(size_t)r * d + c] + y;
                x_add[(size_t)r * d + c] = nx;
                if (out != nullptr) out[(size_t)i * d + c] = from_f32<T>(nx);
            } else {
                out[(size_t)i * d + c] = from_f32<T>(y);
            }
        }
    }
}

// add mode: x [nrows, d] += LN(delta [nrows, d]); h (type `dtype`, may be null) = x.   rows mode: out = LN(x[rows]).
JK_EXPORT int jk_layernorm(const float *src, const int *rows, int nrows, int d, const float *w, const float *b, float eps,
                           float *x_add, void *out, int dtype, cudaStream_t stream) {
    if (nrows == 0) return JK_OK;
    JK_REQUIRE(src && w && nrows > 0 && d > 0, "layernorm: rows %d, width %d", nrows, d);
    JK_REQUIRE(x_add != nullptr || out != nullptr, "layernorm: nothing to write");
    JK_REQUIRE(x_add == nullptr || rows == nullptr, "layernorm: the adding form works on every row");
    JK_REQUIRE((size_t)d * 4 <= 200 * 1024, "layernorm: width %d does not fit shared memory", d);
    const bool vec = d % 4 == 0 && ((uintptr_t)src % 16 == 0) && ((uintptr_t)w % 16 == 0) && (b == nullptr || (uintptr_t)b % 16 == 0) &&
                     (x_add == nullptr || (uintptr_t)x_add % 16 == 0) && (out == nullptr || (uintptr_t)out % 16 == 0);
    const int threads = d >= 4096 ? 512 : (d >= 1024 ? 256 : 128);
    const size_t smem = (size_t)d * sizeof(float);
#define LN_LAUNCH(T, VEC)                                                                                                   \
    do {                                                                                                                    \
        if (smem > 48 * 1024) cudaFuncSetAttribute(layernorm_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        jk_launch(layernorm_kernel<T, VEC>, dim3(nrows), dim3(threads), smem, stream, src, rows, w, b, eps, x_add, (T *)out, d);   \
    } while (0)
    if (dtype == JK_F32) {
        if (vec) LN_LAUNCH(float, true); else LN_LAUNCH(float, false);
    } else if (dtype == JK_BF16) {
        if (vec) LN_LAUNCH(__nv_bfloat16, true); else LN_LAUNCH(__nv_bfloat16, false);
    } else {
        JK_FAIL(JK_UNSUPPORTED, "layernorm: dtype %d", dtype);
    }
#undef LN_LAUNCH
    JK_CHECK_LAUNCH("layernorm");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// out = T(in): the float32 stream as the operand of a product that reads the stream itself.
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void cast_kernel(const float *__restrict__ in, T *__restrict__ out, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = from_f32<T>(in[i]);
}

JK_EXPORT int jk_cast_rows(const float *in, void *out, int dtype, long long n, cudaStream_t stream) {
    if (n == 0) return JK_OK;
    JK_REQUIRE(in && out && n > 0, "cast: nothing to do it with");
    const int blocks = (int)std::min<long long>((n + 255) / 256, 148 * 16);
    if (dtype == JK_F32)
        jk_launch(cast_kernel<float>, dim3(blocks), dim3(256), 0, stream, in, (float *)out, (size_t)n);
    else if (dtype == JK_BF16)
        jk_launch(cast_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, in, (__nv_bfloat16 *)out, (size_t)n);
    else
        JK_FAIL(JK_UNSUPPORTED, "cast: dtype %d", dtype);
    JK_CHECK_LAUNCH("cast");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Gated linear unit: out[t, c] = act(gu[t, c]) * gu[t, di + c], gu float32 [T, 2 di]; act 6: the clamped unit with `limit`.
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void glu_kernel(const float *__restrict__ gu, T *__restrict__ out, int di, size_t total, int act, float limit) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / di, c = i % di;
        const float g = gu[t * 2 * di + c], u = gu[t * 2 * di + di + c];
        if (act == 6) {         // the clamped unit: g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit)
            const float gc = fminf(g, limit), uc = fminf(fmaxf(u, -limit), limit);
            out[i] = from_f32<T>(gc / (1.f + expf(-1.702f * gc)) * (uc + 1.f));
            continue;
        }
        out[i] = from_f32<T>(apply_act(act, g) * u);
    }
}

JK_EXPORT int jk_glu(const float *gu, void *out, int dtype, int ntok, int di, int act, float limit, cudaStream_t stream) {
    if (ntok == 0) return JK_OK;
    JK_REQUIRE(gu && out && ntok > 0 && di > 0, "glu: rows %d, width %d", ntok, di);
    const size_t total = (size_t)ntok * di;
    const int blocks = (int)std::min<size_t>((total + 255) / 256, 148 * 16);
    if (dtype == JK_F32)
        jk_launch(glu_kernel<float>, dim3(blocks), dim3(256), 0, stream, gu, (float *)out, di, total, act, limit);
    else if (dtype == JK_BF16)
        jk_launch(glu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, gu, (__nv_bfloat16 *)out, di, total, act, limit);
    else
        JK_FAIL(JK_UNSUPPORTED, "glu: dtype %d", dtype);
    JK_CHECK_LAUNCH("glu");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Queries, keys and values of a softmax attention whose projections pass a short causal convolution over time, an RMS
// norm over the whole projection (queries and keys) and a rotation of the first `rot_dims` elements of each head:
//     y_t[c]  = sum_j conv[c, j] * u_(t - taps + 1 + j)[c]         u: the projection; zeros before the sequence starts
//     q_t     = rotate(y_t * norm_w / sqrt(mean(y_t^2) + eps))     the mean over all heads' elements at once
//     rotate: (a, b) = elements (2i, 2i+1) of a head, i < rot_dims / 2, at position p:
//             (a cos(p f_i) - b sin(p f_i), b cos(p f_i) + a sin(p f_i)),  the angle p * f_i formed in float32
// The projections before a portion's first row come from the request's tail: the last taps - 1 projected rows of its
// sequence, tail[slot, s, c], s = taps - 2 the newest.  One block per row.  Queries go to q_out [T, nq]; keys (after
// everything) and values (after the convolution) into their pages at the row's position.  `conv_tail_kernel` then
// moves the tails forward; it runs after this kernel has read them.
// ---------------------------------------------------------------------------------------------------------------
struct ConvQkvArgs {
    const float *u;             // [T, ld]
    int ld, q_off, k_off, v_off;
    int nq, nk, nv;             // channels: heads * dk, kv_heads * dk, kv_heads * dv; nk = nv = 0: queries only
    const float *conv_q, *conv_k, *conv_v;      // [channels, taps]; null: no convolution
    const float *norm_q, *norm_k;               // [nq], [nk]; null: no norm
    const float *freq;          // [rot_dims / 2] float32: f_i
    float *tail;                // [slots, taps - 1, nq + nk + nv]
    int taps, dk, dv, kv_heads, rot_dims;
    float eps;
    int rot_half;               // 1: element i < rot_dims / 2 of a head pairs with element i + rot_dims / 2 (else 2i with 2i + 1)
    float rot_mag;              // factor of cos and sin
    int head_norm;              // 1: after the rotation every head of q and k is divided by its root mean square (eps inside);
                                // 2: BEFORE the rotation every head of q and k passes an RMS norm whose weight (norm_q, norm_k:
                                // [dk], shared by the heads) multiplies it; the whole-projection norm is then off
    const float *bias;          // [ld] or null: added to the projection's columns as they are read (no convolution then)
    const int *positions, *row_req, *req_start, *slot_ids, *block_table;
    int max_blocks, page_size;
    void *q_out, *k_pages, *v_pages;
};

template <typename T>
__global__ void conv_qkv_kernel(ConvQkvArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float y[];      // [nq + nk + nv]
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int C = a.nq + a.nk + a.nv;
    const int req = a.row_req[t];
    const int back = t - a.req_start[req];          // rows of this portion before this one
    const int pos = a.positions[t];
    const float *tail = a.tail ? a.tail + (size_t)a.slot_ids[req] * (a.taps - 1) * C : nullptr;
    float ssq = 0.f, ssk = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        int col;
        const float *w;
        if (c < a.nq) { col = a.q_off + c; w = a.conv_q ? a.conv_q + (size_t)c * a.taps : nullptr; }
        else if (c < a.nq + a.nk) { col = a.k_off + c - a.nq; w = a.conv_k ? a.conv_k + (size_t)(c - a.nq) * a.taps : nullptr; }
        else { col = a.v_off + c - a.nq - a.nk; w = a.conv_v ? a.conv_v + (size_t)(c - a.nq - a.nk) * a.taps : nullptr; }
        float acc;
        if (w == nullptr) {
            acc = a.u[(size_t)t * a.ld + col] + (a.bias ? a.bias[col] : 0.f);
        } else {
            acc = 0.f;
            for (int j = 0; j < a.taps; ++j) {
                const int d = a.taps - 1 - j;       // how many rows back
                float uv;
                if (d <= back) uv = a.u[(size_t)(t - d) * a.ld + col];
                else uv = tail[(size_t)(a.taps - 1 + back - d) * C + c];
                acc = fmaf(w[j], uv, acc);
            }
        }
        y[c] = acc;
        if (c < a.nq) ssq += acc * acc;
        else if (c < a.nq + a.nk) ssk += acc * acc;
    }
    const float sum_q = block_sum(ssq, scratch);
    const float sum_k = a.nk > 0 ? block_sum(ssk, scratch) : 0.f;
    const bool whole = a.head_norm != 2;        // the norm over a whole projection
    const float inv_q = (whole && a.norm_q) ? 1.f / sqrtf(sum_q / (float)a.nq + a.eps) : 1.f;
    const float inv_k = (whole && a.norm_k && a.nk > 0) ? 1.f / sqrtf(sum_k / (float)a.nk + a.eps) : 1.f;
    for (int c = threadIdx.x; c < a.nq + a.nk; c += blockDim.x) {
        const bool is_q = c < a.nq;
        const int cc = is_q ? c : c - a.nq;
        const float *nw = whole ? (is_q ? a.norm_q : a.norm_k) : nullptr;
        y[c] = y[c] * (is_q ? inv_q : inv_k) * (nw ? nw[cc] : 1.f);
    }
    __syncthreads();
    // rotation and the stores; a thread reads its partner's element, nobody writes y any more
    T *q_out = (T *)a.q_out + (size_t)t * a.nq;
    const float fpos = (float)pos;
    size_t k_row = 0, v_row = 0;
    if (a.nk > 0) {
        const int page = a.block_table[(size_t)req * a.max_blocks + pos / a.page_size];
        const size_t row = (size_t)page * a.kv_heads * a.page_size + (size_t)(pos % a.page_size);
        k_row = row; v_row = row;
    }
    if (a.head_norm) {
        // a warp per head of q and k: rotate, the head's sum of squares, divide, store
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
        const int half = a.rot_dims >> 1, heads = (a.nq + a.nk) / a.dk;
        for (int hh = warp; hh < heads; hh += nwarp) {
            float *yh = y + (size_t)hh * a.dk;
            if (a.head_norm == 2) {
                // the norm first: the head's mean square, its weight; then the rotation of the normed elements
                const float *nw = hh * a.dk < a.nq ? a.norm_q : a.norm_k;
                float s2 = 0.f;
                for (int e = lane; e < a.dk; e += 32) s2 += yh[e] * yh[e];
                const float inv2 = 1.f / sqrtf(warp_sum(s2) / (float)a.dk + a.eps);
                for (int e = lane; e < a.dk; e += 32) yh[e] = yh[e] * inv2 * (nw ? nw[e] : 1.f);
                __syncwarp();
                for (int e = lane; e < a.dk; e += 32) {
                    float val = yh[e];
                    if (e < a.rot_dims) {
                        const bool first = a.rot_half ? e < half : !(e & 1);
                        const int pair = a.rot_half ? (first ? e : e - half) : e >> 1;
                        const float other = yh[a.rot_half ? (first ? e + half : e - half) : (first ? e + 1 : e - 1)];
                        float sn, cs;
                        sincosf(fpos * a.freq[pair], &sn, &cs);
                        sn *= a.rot_mag; cs *= a.rot_mag;
                        val = first ? val * cs - other * sn : val * cs + other * sn;
                    }
                    const int c = hh * a.dk + e;
                    if (c < a.nq) q_out[c] = from_f32<T>(val);
                    else ((T *)a.k_pages)[(k_row + (size_t)((c - a.nq) / a.dk) * a.page_size) * a.dk + e] = from_f32<T>(val);
                }
                continue;
            }
            float ss = 0.f;
            for (int e = lane; e < a.dk; e += 32) {
                float val = yh[e];
                if (e < a.rot_dims) {
                    const bool first = a.rot_half ? e < half : !(e & 1);
                    const int pair = a.rot_half ? (first ? e : e - half) : e >> 1;
                    const float other = yh[a.rot_half ? (first ? e + half : e - half) : (first ? e + 1 : e - 1)];
                    float sn, cs;
                    sincosf(fpos * a.freq[pair], &sn, &cs);
                    sn *= a.rot_mag; cs *= a.rot_mag;
                    val = first ? val * cs - other * sn : val * cs + other * sn;
                }
                ss += val * val;
            }
            const float inv = 1.f / sqrtf(warp_sum(ss) / (float)a.dk + a.eps);
            for (int e = lane; e < a.dk; e += 32) {
                float val = yh[e];
                if (e < a.rot_dims) {
                    const bool first = a.rot_half ? e < half : !(e & 1);
                    const int pair = a.rot_half ? (first ? e : e - half) : e >> 1;
                    const float other = yh[a.rot_half ? (first ? e + half : e - half) : (first ? e + 1 : e - 1)];
                    float sn, cs;
                    sincosf(fpos * a.freq[pair], &sn, &cs);
                    sn *= a.rot_mag; cs *= a.rot_mag;
                    val = first ? val * cs - other * sn : val * cs + other * sn;
                }
                const int c = hh * a.dk + e;
                if (c < a.nq) q_out[c] = from_f32<T>(val * inv);
                else ((T *)a.k_pages)[(k_row + (size_t)((c - a.nq) / a.dk) * a.page_size) * a.dk + e] = from_f32<T>(val * inv);
            }
        }
    }
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        if (c < a.nq + a.nk) {
            if (a.head_norm) continue;
            const bool is_q = c < a.nq;
            const int cc = is_q ? c : c - a.nq;
            const int head = cc / a.dk, e = cc % a.dk;
            float val = y[c];
            if (e < a.rot_dims) {
                const int half = a.rot_dims >> 1;
                const bool first = a.rot_half ? e < half : !(e & 1);
                const int pair = a.rot_half ? (first ? e : e - half) : e >> 1;
                const float ang = fpos * a.freq[pair];
                float sn, cs;
                sincosf(ang, &sn, &cs);
                sn *= a.rot_mag; cs *= a.rot_mag;
                const float other = y[a.rot_half ? (first ? c + half : c - half) : (first ? c + 1 : c - 1)];
                val = first ? fmaf(val, cs, -other * sn) : fmaf(val, cs, other * sn);
            }
            if (is_q) q_out[cc] = from_f32<T>(val);
            else ((T *)a.k_pages)[(k_row + (size_t)head * a.page_size) * a.dk + e] = from_f32<T>(val);
        } else {
            const int cc = c - a.nq - a.nk;
            const int head = cc / a.dv, e = cc % a.dv;
            ((T *)a.v_pages)[(v_row + (size_t)head * a.page_size) * a.dv + e] = from_f32<T>(y[c]);
        }
    }
}

// tail[slot, s, c] <- the projection taps - 1 - s rows before the end of the request's sequence after this step.
// One thread per (request, channel); it reads every old entry it needs before it overwrites it (ascending s reads
// ahead of the writes).
__global__ void conv_tail_kernel(ConvQkvArgs a, int nreq) {
    pdl_trigger();
    pdl_wait();
    const int C = a.nq + a.nk + a.nv;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nreq * C) return;
    const int req = idx / C, c = idx % C;
    const int first = a.req_start[req], n = a.req_start[req + 1] - first;
    int col;
    if (c < a.nq) col = a.q_off + c;
    else if (c < a.nq + a.nk) col = a.k_off + c - a.nq;
    else col = a.v_off + c - a.nq - a.nk;
    float *tail = a.tail + (size_t)a.slot_ids[req] * (a.taps - 1) * C;
    for (int s = 0; s < a.taps - 1; ++s) {
        const int off = n - (a.taps - 1) + s;       // row of this portion (negative: before it)
        const float v = off >= 0 ? a.u[(size_t)(first + off) * a.ld + col] : tail[(size_t)(s + n) * C + c];
        tail[(size_t)s * C + c] = v;
    }
}

JK_EXPORT int jk_conv_qkv(const float *u, int ld, int q_off, int k_off, int v_off, int heads, int kv_heads, int dk, int dv,
                          int has_kv, const float *conv_q, const float *conv_k, const float *conv_v, int taps,
                          const float *norm_q, const float *norm_k, float eps, const float *freq, int rot_dims, float *tail,
                          const int *positions, const int *row_req, const int *req_start, const int *slot_ids,
                          const int *block_table, int max_blocks, int page_size, void *q_out, void *k_pages, void *v_pages,
                          int dtype, int T, int nreq, int rot_half, float rot_mag, int head_norm, const float *bias, cudaStream_t stream) {
    if (T == 0) return JK_OK;
    ConvQkvArgs a;
    a.bias = bias;
    a.u = u; a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
    a.nq = heads * dk; a.nk = has_kv ? kv_heads * dk : 0; a.nv = has_kv ? kv_heads * dv : 0;
    a.conv_q = conv_q; a.conv_k = conv_k; a.conv_v = conv_v; a.norm_q = norm_q; a.norm_k = norm_k; a.freq = freq; a.tail = tail;
    a.taps = taps; a.dk = dk; a.dv = dv; a.kv_heads = kv_heads; a.rot_dims = rot_dims; a.eps = eps;
    a.rot_half = rot_half; a.rot_mag = rot_mag > 0.f ? rot_mag : 1.f; a.head_norm = head_norm;
    a.positions = positions; a.row_req = row_req; a.req_start = req_start; a.slot_ids = slot_ids; a.block_table = block_table;
    a.max_blocks = max_blocks; a.page_size = page_size; a.q_out = q_out; a.k_pages = k_pages; a.v_pages = v_pages;
    const bool conv = conv_q || conv_k || conv_v;
    JK_REQUIRE(u && q_out && positions && row_req && req_start && heads > 0 && dk > 0, "conv_qkv: an argument is missing");
    JK_REQUIRE(!has_kv || (k_pages && v_pages && block_table && kv_heads > 0 && dv > 0 && page_size > 0), "conv_qkv: keys without a cache");
    JK_REQUIRE(!(conv && bias), "conv_qkv: a bias with a convolution is not built");
    JK_REQUIRE(!conv || (taps >= 1 && (taps == 1 || (tail && slot_ids))), "conv_qkv: a convolution of %d taps without its tails", taps);
    JK_REQUIRE(rot_dims >= 0 && rot_dims <= dk && rot_dims % 2 == 0 && (rot_dims == 0 || freq), "conv_qkv: rotation of %d of %d elements", rot_dims, dk);
    const int C = a.nq + a.nk + a.nv;
    const size_t smem = (size_t)C * sizeof(float);
    JK_REQUIRE(smem <= 200 * 1024, "conv_qkv: %d channels do not fit shared memory", C);
    // a step of few rows has few blocks: more threads a row then, so that a thread's chain of channels is short
    int threads = C >= 2048 ? 512 : (C >= 512 ? 256 : 128);
    if (T <= 64) threads = std::min(1024, std::max(threads, (C / 2 + 31) / 32 * 32));
    if (dtype == JK_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(conv_qkv_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        jk_launch(conv_qkv_kernel<float>, dim3(T), dim3(threads), smem, stream, a);
    } else if (dtype == JK_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(conv_qkv_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        jk_launch(conv_qkv_kernel<__nv_bfloat16>, dim3(T), dim3(threads), smem, stream, a);
    } else {
        JK_FAIL(JK_UNSUPPORTED, "conv_qkv: dtype %d", dtype);
    }
    JK_CHECK_LAUNCH("conv_qkv");
    if (conv && taps > 1) {
        const int total = nreq * C;
        jk_launch(conv_tail_kernel, dim3((total + 127) / 128), dim3(128), 0, stream, a, nreq);
        JK_CHECK_LAUNCH("conv_tail");
    }
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Linear attention as a recurrence over a request's rows, per head:
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T        S: [dk, dv] float32, carried in state[slot, head]
//     o_t = S_t^T q_t
// q, k, v pass `qkv_act` (none or silu); q is multiplied by q_scale.  The decay a_t [dk] is either one constant per head
// (decay[head], for all channels and rows) or projected: z = W2 r_t + b2 with r_t the `rank` columns of the fused
// product at r_off, a = exp(log_sigmoid(z) / tau), all in float32 (W2 may be stored as bfloat16).
// A block of the scan kernel owns (head, work item, a slice of value columns) and walks the item's rows in order.  Its
// threads are (column, part): `kq` neighbouring lanes share a column of S, lane `part` keeping the key channels part,
// part + kq, part + 2 kq ... in registers; a row's output is the lanes' partial sums added by shuffles.  Rows are staged
// through shared memory a chunk at a time (activations applied, decays formed there, once per block), so a row costs no
// block barrier; the state is read and written once per item.
//
// Work items.  A request that brings at most SCAN_PIECE rows is one item: from its state slot, through its rows, back into
// the slot ("direct").  A longer portion is cut into pieces of SCAN_PIECE rows that run side by side, each from a state of
// zeros: a piece leaves its rows' outputs without what came before the piece, its own end state in `piece_state`, and (for
// a projected decay) the running product of the decays since the piece's start, b_t, in `cum`.  `scan_carry_kernel` then
// walks each such request's pieces in order, S <- diag(b_end) S + S_piece, leaving in `piece_state` the state at each piece's
// START and in the slot the state after the last; `scan_prefix_kernel` adds (q_t * b_t)^T S_start to the piece's rows.
// Nothing is ever divided by a decay.  The order of the sums of a row depends on where its piece starts (every SCAN_PIECE
// rows from the start of its portion) and on nothing else of the batch.
// ---------------------------------------------------------------------------------------------------------------
constexpr int SCAN_PIECE = jk::SCAN_PIECE;

struct ScanArgs {
    const float *u;             // [T, ld]
    int ld, q_off, k_off, v_off, r_off;
    int heads, dk, dv, qkv_act;
    float q_scale;
    const float *decay;         // [heads] or null
    const void *w2;             // [heads * dk, rank] (TW: float or bfloat16) or null
    const float *b2;            // [heads * dk] or null
    int rank;
    float inv_tau;
    float *state;               // [slots, heads, dk, dv]
    const int *req_start, *slot_ids;
    float *out;                 // [T, heads * dv] float32
    int kq;                     // lanes that share a column (a power of two up to 32)
    int chunk;                  // rows staged at a time
    const int *direct;          // [n_direct] requests that run as one item (null: requests 0 .. n_direct-1)
    int n_direct;
    const int *pieces;          // [n_pieces, 2] (first row, rows)
    int n_pieces;
    const int *piece_reqs;      // [n_piece_reqs, 3] (request, its first piece, its pieces)
    float *piece_state;         // [n_pieces, heads, dk, dv]
    float *cum;                 // [T, heads, dk] running products of a projected decay inside each piece
    int vec4;                   // 1: rows, offsets and sizes are multiples of four floats: staging moves 16 bytes at a time
    int dkp;                    // channels of a staged row: dk rounded up to kq * KS; the padding stays zero, so the scan's
                                // inner loop needs no bounds
    // The form in which a row reads the state BEFORE its own decay, with a bonus for its own key:
    //     o_t = (S_(t-1) + diag(bonus) k_t v_t^T)^T q_t,  then  S_t = diag(a_t) S_(t-1) + k_t v_t^T
    // (bonus [heads, dk]; null: the form above, o_t = S_t^T q_t).  The running product that the prefix kernel multiplies a
    // row's query by is then the one up to the row BEFORE it.
    const float *bonus;
    int decay_form;             // projected decay: 0 sigmoid(z)^(1/tau), 1 exp(-exp(z))
    int rank_act;               // MixAct on the decay projection's `rank` columns before W2
    int stage_w2;               // 1: the head's rows of W2 lie in shared memory, transposed ([rank, dk + 1] float32)
};

constexpr int SCAN_THREADS = 256;     // (column pair, part) threads: a row staged once serves 128 columns at four lanes a column
// SCAN_CPT: columns of S a thread keeps; what it reads of a row's q, k and decay serves them all.  Four where portions run
// as pieces (the shared-memory reads bound the scan), two in steps of short requests (more blocks, shorter threads).
// Threads that keep little state leave registers for more blocks an SM: the rows' dependent steps need warps to hide behind.
// PROJ: the decay is projected (the instances for a constant decay carry none of that code, nor its registers).
// OCC: blocks an SM that the registers must allow: three where portions run as pieces of many rows (more warps to hide a
// row's dependent steps behind), two in steps of few rows (a thread's loads all in flight, nothing spilled).
template <typename TW, int KS, int SCAN_CPT, bool PROJ, int OCC = 2>      // KS: key channels per thread
__global__ void __launch_bounds__(SCAN_THREADS, OCC)
linear_scan_kernel(ScanArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    const int kq = a.kq, cols = SCAN_THREADS / kq * SCAN_CPT, dk = a.dk;
    const int head = blockIdx.x, item = blockIdx.y, c0 = blockIdx.z * cols;
    const int dkp = a.dkp;
    float4 *sx = reinterpret_cast<float4 *>(sm);        // [chunk, dkp] (decay, k, q, -) of a row's channel, side by side
    float *sv = sm + 4 * (size_t)a.chunk * dkp;         // [chunk, cols]
    float *sr = sv + (size_t)a.chunk * cols;            // [chunk, rank]
    float *sw = sr + (size_t)a.chunk * a.rank;          // [rank, dk + 1]: the head's rows of W2, transposed (stage_w2)
    // within a warp the column groups vary fastest, so that lanes with one part read neighbouring columns of a state row
    const int per_warp = 32 / kq, lane = threadIdx.x & 31;
    const int col = ((threadIdx.x >> 5) * per_warp + lane % per_warp) * SCAN_CPT, part = lane / per_warp;
    bool live[SCAN_CPT];
#pragma unroll
    for (int c = 0; c < SCAN_CPT; ++c) live[c] = c0 + col + c < a.dv;
    int first, last;
    float *S;
    const bool piece = item >= a.n_direct;
    if (!piece) {
        const int req = a.direct ? a.direct[item] : item;
        first = a.req_start[req]; last = a.req_start[req + 1];
        S = a.state + (((size_t)a.slot_ids[req] * a.heads + head) * dk) * a.dv + c0 + col;
    } else {
        const int p = item - a.n_direct;
        first = a.pieces[2 * p]; last = first + a.pieces[2 * p + 1];
        S = a.piece_state + (((size_t)p * a.heads + head) * dk) * a.dv + c0 + col;
    }
    float s[SCAN_CPT][KS];
#pragma unroll
    for (int c = 0; c < SCAN_CPT; ++c)
#pragma unroll
        for (int i = 0; i < KS; ++i) s[c][i] = (!piece && live[c] && part + i * kq < dk) ? S[(size_t)(part + i * kq) * a.dv + c] : 0.f;
    const float head_decay = a.decay ? a.decay[head] : 1.f;
    const bool with_bonus = a.bonus != nullptr;
    const bool write_cum = PROJ && piece && blockIdx.z == 0;
    if (dkp > dk)       // the padding channels: zero once, nothing writes them afterwards
        for (int i = threadIdx.x; i < a.chunk * dkp; i += SCAN_THREADS) sx[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (PROJ && a.stage_w2) {   // read along W2's rows, kept so that threads with neighbouring channels read neighbouring words
        const TW *w = (const TW *)a.w2 + (size_t)head * dk * a.rank;
        for (int i = threadIdx.x; i < dk * a.rank; i += SCAN_THREADS) {
            const int kk = i / a.rank, r = i - kk * a.rank;
            sw[r * (dk + 1) + kk] = to_f32(w[i]);
        }
    }
    for (int t0 = first; t0 < last; t0 += a.chunk) {
        const int n = min(a.chunk, last - t0);
        __syncthreads();            // the chunk before has been read
        if (PROJ)
            for (int i = threadIdx.x; i < n * a.rank; i += SCAN_THREADS) {
                const int tt = i / a.rank;
                sr[i] = apply_act(a.rank_act, a.u[(size_t)(t0 + tt) * a.ld + a.r_off + (i - tt * a.rank)]);
            }
        if (a.vec4) {
            // four neighbouring channels of a row at a time, all of a thread's loads ahead of the arithmetic
            for (int i0 = threadIdx.x * 4; i0 < n * dk; i0 += 8 * SCAN_THREADS) {
                float4 qv[2], kv[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = i0 + j * 4 * SCAN_THREADS;
                    if (i < n * dk) {
                        const int tt = i / dk, kk = i - tt * dk;
                        const float *row = a.u + (size_t)(t0 + tt) * a.ld + head * dk + kk;
                        qv[j] = *reinterpret_cast<const float4 *>(row + a.q_off);
                        kv[j] = *reinterpret_cast<const float4 *>(row + a.k_off);
                    }
                }
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = i0 + j * 4 * SCAN_THREADS;
                    if (i < n * dk) {
                        const float qq[4] = {qv[j].x, qv[j].y, qv[j].z, qv[j].w}, kk4[4] = {kv[j].x, kv[j].y, kv[j].z, kv[j].w};
                        const int at = (i / dk) * dkp + i % dk;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            sx[at + e].y = apply_act(a.qkv_act, kk4[e]);
                            sx[at + e].z = apply_act(a.qkv_act, qq[e]) * a.q_scale;
                            if (!PROJ) sx[at + e].x = head_decay;
                            if (a.bonus != nullptr) sx[at + e].w = a.bonus[head * dk + i % dk + e];
                        }
                    }
                }
            }
        } else {
            // four elements a thread at a time, their loads ahead of the arithmetic
            for (int i0 = threadIdx.x; i0 < n * dk; i0 += 4 * SCAN_THREADS) {
                float qv[4], kv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + j * SCAN_THREADS;
                    if (i < n * dk) {
                        const int tt = i / dk, kk = i - tt * dk;
                        const float *row = a.u + (size_t)(t0 + tt) * a.ld;
                        qv[j] = row[a.q_off + head * dk + kk];
                        kv[j] = row[a.k_off + head * dk + kk];
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + j * SCAN_THREADS;
                    if (i < n * dk) {
                        const int at = (i / dk) * dkp + i % dk;
                        sx[at].y = apply_act(a.qkv_act, kv[j]);
                        sx[at].z = apply_act(a.qkv_act, qv[j]) * a.q_scale;
                        if (!PROJ) sx[at].x = head_decay;
                        if (a.bonus != nullptr) sx[at].w = a.bonus[head * dk + i % dk];
                    }
                }
            }
        }
        for (int i = threadIdx.x; i < n * cols; i += SCAN_THREADS) {
            const int tt = i / cols, cc = i - tt * cols;
            sv[i] = c0 + cc < a.dv ? apply_act(a.qkv_act, a.u[(size_t)(t0 + tt) * a.ld + a.v_off + head * a.dv + c0 + cc]) : 0.f;
        }
        __syncthreads();
        if (PROJ && a.stage_w2) {
            // a thread forms the decays of one channel in four rows: a word of W2 serves four products.  Every decay is the
            // same chain of sums as below, in the order of W2's columns.
            const int groups = (n + 3) / 4;
            for (int i = threadIdx.x; i < groups * dk; i += SCAN_THREADS) {
                const int tg = i / dk, kk = i - tg * dk, tt0 = tg * 4;
                const float bias = a.b2 ? a.b2[head * dk + kk] : 0.f;
                float z[4] = {bias, bias, bias, bias};
                const float *r0 = sr + (size_t)tt0 * a.rank;
                const float *r1 = sr + (size_t)min(tt0 + 1, n - 1) * a.rank;
                const float *r2 = sr + (size_t)min(tt0 + 2, n - 1) * a.rank;
                const float *r3 = sr + (size_t)min(tt0 + 3, n - 1) * a.rank;
                const float *w = sw + kk;
                int r = 0;
                // four columns of a staged row in one read, where a thread's state leaves the registers for it
                if (KS * SCAN_CPT <= 16 && a.rank % 4 == 0 && (a.chunk * cols) % 4 == 0) {
                    for (; r < a.rank; r += 4) {
                        const float4 x0 = *reinterpret_cast<const float4 *>(r0 + r), x1 = *reinterpret_cast<const float4 *>(r1 + r);
                        const float4 x2 = *reinterpret_cast<const float4 *>(r2 + r), x3 = *reinterpret_cast<const float4 *>(r3 + r);
                        const float w0 = w[r * (dk + 1)], w1 = w[(r + 1) * (dk + 1)], w2v = w[(r + 2) * (dk + 1)], w3 = w[(r + 3) * (dk + 1)];
                        z[0] = fmaf(w3, x0.w, fmaf(w2v, x0.z, fmaf(w1, x0.y, fmaf(w0, x0.x, z[0]))));
                        z[1] = fmaf(w3, x1.w, fmaf(w2v, x1.z, fmaf(w1, x1.y, fmaf(w0, x1.x, z[1]))));
                        z[2] = fmaf(w3, x2.w, fmaf(w2v, x2.z, fmaf(w1, x2.y, fmaf(w0, x2.x, z[2]))));
                        z[3] = fmaf(w3, x3.w, fmaf(w2v, x3.z, fmaf(w1, x3.y, fmaf(w0, x3.x, z[3]))));
                    }
                }
                for (; r < a.rank; ++r) {
                    const float wv = w[r * (dk + 1)];
                    z[0] = fmaf(wv, r0[r], z[0]);
                    z[1] = fmaf(wv, r1[r], z[1]);
                    z[2] = fmaf(wv, r2[r], z[2]);
                    z[3] = fmaf(wv, r3[r], z[3]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (tt0 + j < n)
                        sx[(tt0 + j) * dkp + kk].x = a.decay_form == 1 ? expf(-expf(z[j])) : expf(log_sigmoid_f(z[j]) * a.inv_tau);
            }
            __syncthreads();
        } else if (PROJ) {
            for (int i = threadIdx.x; i < n * dk; i += SCAN_THREADS) {
                const int tt = i / dk, kk = i - tt * dk;
                const TW *w = (const TW *)a.w2 + (size_t)(head * dk + kk) * a.rank;
                float z = a.b2 ? a.b2[head * dk + kk] : 0.f;
                for (int r = 0; r < a.rank; ++r) z = fmaf(to_f32(w[r]), sr[tt * a.rank + r], z);
                sx[tt * dkp + kk].x = a.decay_form == 1 ? expf(-expf(z)) : expf(log_sigmoid_f(z) * a.inv_tau);
            }
            __syncthreads();
        }
        if (write_cum) {            // b_t = a_t * b_(t-1) per channel, from the piece's start
            for (int kk = threadIdx.x; kk < dk; kk += SCAN_THREADS) {
                float b = t0 > first ? a.cum[((size_t)(t0 - 1) * a.heads + head) * dk + kk] : 1.f;
                for (int tt = 0; tt < n; ++tt) {
                    b *= sx[tt * dkp + kk].x;
                    a.cum[((size_t)(t0 + tt) * a.heads + head) * dk + kk] = b;
                }
            }
        }
        for (int tt = 0; tt < n; ++tt) {
            float vv[SCAN_CPT], o[SCAN_CPT][2];
#pragma unroll
            for (int c = 0; c < SCAN_CPT; ++c) { vv[c] = sv[tt * cols + col + c]; o[c][0] = o[c][1] = 0.f; }
            const float4 *x = sx + (size_t)tt * dkp + part;
#pragma unroll
            for (int i = 0; i < KS; ++i) {          // no bounds: a staged row is padded with zeros up to kq * KS channels
                const float4 e = x[i * kq];
#pragma unroll
                for (int c = 0; c < SCAN_CPT; ++c) {
                    if (with_bonus) {       // the row reads the state as the row before left it, its own key with the bonus
                        const float kv = e.y * vv[c];
                        o[c][i & 1] = fmaf(fmaf(e.w, kv, s[c][i]), e.z, o[c][i & 1]);
                        s[c][i] = fmaf(e.x, s[c][i], kv);
                    } else {
                        s[c][i] = fmaf(e.x, s[c][i], e.y * vv[c]);
                        o[c][i & 1] = fmaf(s[c][i], e.z, o[c][i & 1]);
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < SCAN_CPT; ++c) {
                float sum = o[c][0] + o[c][1];
                for (int off = kq >> 1; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off * per_warp);
                if (part == 0 && live[c]) a.out[(size_t)(t0 + tt) * a.heads * a.dv + head * a.dv + c0 + col + c] = sum;
            }
        }
    }
#pragma unroll
    for (int c = 0; c < SCAN_CPT; ++c)
        if (live[c]) {
#pragma unroll
            for (int i = 0; i < KS; ++i)
                if (part + i * kq < dk) S[(size_t)(part + i * kq) * a.dv + c] = s[c][i];
        }
}

// One thread per (request with pieces, head, element of S): the pieces in order.  What a piece brings (its end state and
// its decay) does not depend on the running state, so the loads of eight pieces go out before the chain uses them.
__global__ void scan_carry_kernel(ScanArgs a) {
    pdl_trigger();
    pdl_wait();
    const int head = blockIdx.y;
    const int *pr = a.piece_reqs + 3 * blockIdx.z;
    const int req = pr[0], p0 = pr[1], np = pr[2];
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= a.dk * a.dv) return;
    const int kk = e / a.dv;
    const size_t stride = (size_t)a.heads * a.dk * a.dv;
    float *slot = a.state + ((size_t)a.slot_ids[req] * a.heads + head) * a.dk * a.dv + e;
    float *ps = a.piece_state + ((size_t)p0 * a.heads + head) * a.dk * a.dv + e;
    float run = *slot;
    // a constant decay to the power of a whole piece's rows (every piece but the last has that many)
    float d_whole = 1.f;
    if (a.w2 == nullptr) {
        const float hd = a.decay[head];
        for (int i = 0; i < SCAN_PIECE; ++i) d_whole *= hd;
    }
    for (int b0 = 0; b0 < np; b0 += 8) {
        float mine[8], d[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int p = b0 + j;
            if (p < np) {
                mine[j] = ps[(size_t)p * stride];
                const int first = a.pieces[2 * (p0 + p)], n = a.pieces[2 * (p0 + p) + 1];
                if (a.w2 != nullptr) {
                    d[j] = a.cum[((size_t)(first + n - 1) * a.heads + head) * a.dk + kk];
                } else if (n == SCAN_PIECE) {
                    d[j] = d_whole;
                } else {
                    const float hd = a.decay[head];
                    float x = 1.f;
                    for (int i = 0; i < n; ++i) x *= hd;
                    d[j] = x;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int p = b0 + j;
            if (p < np) {
                ps[(size_t)p * stride] = run;          // the state at the piece's start
                run = fmaf(d[j], run, mine[j]);
            }
        }
    }
    *slot = run;
}

// out[t, head, v] += sum_k q_t[k] b_t[k] S_start[k, v] for the rows of a piece: a float32 product of [rows, dk] by
// [dk, dv] per piece and head.  A block owns (piece, head, 128 columns; 64 for narrower heads): S_start's slice and the piece's rows of q * b
// (transposed) lie in shared memory; thread (ty, tx) of 8 x 16 keeps an 8 x 8 tile of the result in registers (rows
// ty * 4 + {0..3} and 32 + ty * 4 + {0..3}, columns tx * 4 + {0..3} and 64 + tx * 4 + {0..3}), so that a step of k costs
// four 16-byte reads for 64 products.
constexpr int PFX_COLS = 128, PFX_ROWS = SCAN_PIECE, PFX_K = 128;
static_assert(PFX_ROWS == 64, "the prefix kernel's tiles are written for pieces of 64 rows");
// Shared memory for blocks of `cols` columns and heads of dk key channels: no more steps of k than a head has.
static size_t pfx_smem(int cols, int dk) { return sizeof(float) * (size_t)std::min(dk, PFX_K) * (cols + PFX_ROWS); }

// COLS: 128, or 64 for heads of at most 64 values (a thread then keeps 8 x 4 results, and a block half the memory).
template <int COLS>
__global__ void __launch_bounds__(128)
scan_prefix_kernel(ScanArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int CW = COLS / 16;               // columns a thread: two runs of four, or one
    extern __shared__ __align__(16) float pfx_sm[];
    const int kstep = min(a.dk, PFX_K);
    float *Ssm = pfx_sm;                        // [kstep, COLS]
    float *qb = pfx_sm + kstep * COLS;          // [kstep, PFX_ROWS]
    __shared__ float pw[SCAN_PIECE];            // a constant decay to the powers 1 .. SCAN_PIECE, by the carry's own products
    const int p = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * COLS;
    const int first = a.pieces[2 * p], n = a.pieces[2 * p + 1];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const float *S = a.piece_state + ((size_t)p * a.heads + head) * a.dk * a.dv;
    if (a.w2 == nullptr && threadIdx.x < SCAN_PIECE) {
        const float hd = a.decay[head];
        float b = hd;
        for (int j = 0; j < threadIdx.x; ++j) b *= hd;
        pw[threadIdx.x] = b;
    }
    float acc[8][CW];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int c = 0; c < CW; ++c) acc[r][c] = 0.f;
    for (int k0 = 0; k0 < a.dk; k0 += kstep) {
        const int nk = min(kstep, a.dk - k0);
        __syncthreads();
        if (a.vec4 && c0 + COLS <= a.dv) {
            for (int i = threadIdx.x * 4; i < nk * COLS; i += 128 * 4) {
                const int kk = i / COLS, cc = i - kk * COLS;
                *reinterpret_cast<float4 *>(Ssm + i) = *reinterpret_cast<const float4 *>(S + (size_t)(k0 + kk) * a.dv + c0 + cc);
            }
        } else {
            for (int i = threadIdx.x; i < nk * COLS; i += 128) {
                const int kk = i / COLS, cc = i - kk * COLS;
                Ssm[i] = c0 + cc < a.dv ? S[(size_t)(k0 + kk) * a.dv + c0 + cc] : 0.f;
            }
        }
        // q * b of the piece's rows, transposed; rows beyond the piece's end are zeros
        for (int i = threadIdx.x; i < PFX_ROWS * nk; i += 128) {
            const int tt = i / nk, kk = i - tt * nk;
            float val = 0.f;
            if (tt < n) {
                const int t = first + tt;
                float b;
                if (a.bonus == nullptr) b = a.w2 != nullptr ? a.cum[((size_t)t * a.heads + head) * a.dk + k0 + kk] : pw[tt];
                else if (tt == 0) b = 1.f;        // the decays up to the row before: none at the piece's first row
                else b = a.w2 != nullptr ? a.cum[((size_t)(t - 1) * a.heads + head) * a.dk + k0 + kk] : pw[tt - 1];
                val = apply_act(a.qkv_act, a.u[(size_t)t * a.ld + a.q_off + head * a.dk + k0 + kk]) * a.q_scale * b;
            }
            qb[kk * PFX_ROWS + tt] = val;
        }
        __syncthreads();
        for (int kk = 0; kk < nk; ++kk) {
            const float4 r0 = *reinterpret_cast<const float4 *>(qb + kk * PFX_ROWS + ty * 4);
            const float4 r1 = *reinterpret_cast<const float4 *>(qb + kk * PFX_ROWS + 32 + ty * 4);
            const float rv[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
            float cv[CW];
            const float4 s0 = *reinterpret_cast<const float4 *>(Ssm + kk * COLS + tx * 4);
            cv[0] = s0.x; cv[1] = s0.y; cv[2] = s0.z; cv[3] = s0.w;
            if (CW == 8) {
                const float4 s1 = *reinterpret_cast<const float4 *>(Ssm + kk * COLS + 64 + tx * 4);
                cv[CW - 4] = s1.x; cv[CW - 3] = s1.y; cv[CW - 2] = s1.z; cv[CW - 1] = s1.w;
            }
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int c = 0; c < CW; ++c) acc[r][c] = fmaf(rv[r], cv[c], acc[r][c]);
        }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const int tt = (r < 4 ? 0 : 32) + ty * 4 + (r & 3);
        if (tt >= n) continue;
        float *o = a.out + (size_t)(first + tt) * a.heads * a.dv + head * a.dv + c0;
#pragma unroll
        for (int c = 0; c < CW; ++c) {
            const int cc = (c < 4 ? 0 : 64) + tx * 4 + (c & 3);
            if (c0 + cc < a.dv) o[cc] += acc[r][c];
        }
    }
}

// Rows of scratch the pieces of a step of `rows` rows need at most: piece_state floats, cum floats.
JK_EXPORT long long jk_linear_scan_scratch_floats(int rows, int heads, int dk, int dv, int projected) {
    return jk::scan_scratch_floats(rows, heads, dk, dv, projected != 0);
}
JK_EXPORT int jk_linear_scan_piece() { return SCAN_PIECE; }

JK_EXPORT int jk_linear_scan(const float *u, int ld, int q_off, int k_off, int v_off, int heads, int dk, int dv, int qkv_act,
                             float q_scale, const float *decay, const void *w2, int w2_dtype, const float *b2, int r_off, int rank,
                             float tau, float *state, const int *req_start, const int *slot_ids, int nreq, int T, float *out,
                             const int *direct, int n_direct, const int *pieces, int n_pieces, const int *piece_reqs,
                             int n_piece_reqs, float *scratch, long long scratch_floats, int sms, const float *bonus, int decay_form,
                             int rank_act, cudaStream_t stream) {
    if (T == 0 || nreq == 0) return JK_OK;
    JK_REQUIRE(u && state && req_start && slot_ids && out && heads > 0 && dk > 0 && dv > 0, "linear_scan: an argument is missing");
    JK_REQUIRE((decay != nullptr) != (w2 != nullptr), "linear_scan: the decay is a constant per head or projected, one of the two");
    JK_REQUIRE(w2 == nullptr || (rank > 0 && (tau > 0.f || decay_form == 1)), "linear_scan: a projected decay of rank %d, tau %g", rank, tau);
    JK_REQUIRE(dk <= 2048, "linear_scan: %d key channels a head exceed 2048", dk);
    if (n_pieces == 0 && direct == nullptr && n_direct <= 0) n_direct = nreq;        // no lists: every request is one item
    JK_REQUIRE(n_direct >= 0 && n_pieces >= 0 && n_direct + n_pieces > 0, "linear_scan: nothing to do");
    JK_REQUIRE(n_pieces == 0 || (pieces && piece_reqs && n_piece_reqs > 0 && scratch), "linear_scan: pieces without their lists or scratch");
    const long long state_floats = (long long)n_pieces * heads * dk * dv;
    JK_REQUIRE(n_pieces == 0 || state_floats + (w2 ? (long long)T * heads * dk : 0) <= scratch_floats,
               "linear_scan: %d pieces need more scratch than %lld floats", n_pieces, scratch_floats);
    // lanes per column: as few as keep a thread's state at 64 values (more beyond 1024 and 512 channels); more of them,
    // and so fewer columns a block and more blocks, while the blocks do not fill the SMs
    const int sm_count = sms > 0 ? sms : 148;
    const int items = n_direct + n_pieces;
    auto lanes_for = [&](int c) {
        int q = 1;
        while (q < 32 && (dk + q - 1) / q > 64 / c) q *= 2;
        return q;
    };
    int cpt = n_pieces > 0 ? 4 : 2;
    int kq = lanes_for(cpt);
    // a block's columns beyond a head's values are idle threads: fewer columns a thread first, then more lanes a column
    if (cpt == 4 && SCAN_THREADS / kq * cpt > dv) {
        cpt = 2;
        kq = lanes_for(cpt);
    }
    while (kq < 32 && 2 * kq <= dk && SCAN_THREADS / kq * cpt > dv) kq *= 2;
    while (kq < 32 && 2 * kq <= dk && (long long)heads * items * ((dv + SCAN_THREADS / kq * cpt - 1) / (SCAN_THREADS / kq * cpt)) < sm_count)
        kq *= 2;
    const int cols = SCAN_THREADS / kq * cpt;
    const int per_thread = (dk + kq - 1) / kq;
    int ks = 1;
    while (ks < per_thread) ks *= 2;            // the instance's channels a thread (below)
    const int dkp = kq * ks;
    const size_t row_bytes = sizeof(float) * (4 * (size_t)dkp + cols + (w2 ? rank : 0));
    int chunk = (int)std::min<size_t>(32, std::max<size_t>(1, (40 * 1024) / row_bytes));
    chunk = std::min(chunk, T);
    // the head's rows of W2 beside the staged rows, while they fit: read once per block along their rows
    const size_t w2_bytes = w2 ? sizeof(float) * (size_t)rank * (dk + 1) : 0;
    const int stage_w2 = w2 != nullptr && w2_bytes <= 64 * 1024 ? 1 : 0;
    ScanArgs a{u, ld, q_off, k_off, v_off, r_off, heads, dk, dv, qkv_act, q_scale, decay, w2, b2, rank, tau > 0.f ? 1.f / tau : 0.f,
               state, req_start, slot_ids, out, kq, chunk, direct, n_direct, pieces, n_pieces, piece_reqs, scratch,
               scratch ? scratch + state_floats : nullptr,
               (dk % 4 == 0 && dv % 4 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && (uintptr_t)u % 16 == 0 &&
                (scratch == nullptr || (uintptr_t)scratch % 16 == 0)) ? 1 : 0,
               dkp, bonus, decay_form, rank_act, stage_w2};
    dim3 grid(heads, items, (dv + cols - 1) / cols);
    JK_REQUIRE(items <= 65535 && grid.z <= 65535 && heads <= 65535, "linear_scan: %d items in one launch", items);
    const size_t smem = row_bytes * chunk + (stage_w2 ? w2_bytes : 0);
#define SCAN_LAUNCH_O(TW, KS, C, P, O)                                                                                          \
    do {                                                                                                                        \
        if (smem > 48 * 1024)                                                                                                   \
            cudaFuncSetAttribute(linear_scan_kernel<TW, KS, C, P, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        jk_launch(linear_scan_kernel<TW, KS, C, P, O>, grid, dim3(SCAN_THREADS), smem, stream, a);                              \
    } while (0)
#define SCAN_LAUNCH_C(TW, KS, C, P)                                         \
    do {                                                                    \
        if constexpr (KS * C <= 16) {                                       \
            if (n_pieces > 0) SCAN_LAUNCH_O(TW, KS, C, P, 3);               \
            else SCAN_LAUNCH_O(TW, KS, C, P, 2);                            \
        } else {                                                            \
            SCAN_LAUNCH_O(TW, KS, C, P, 2);                                 \
        }                                                                   \
    } while (0)
#define SCAN_LAUNCH(TW, KS, P)                      \
    do {                                            \
        if (cpt == 4) SCAN_LAUNCH_C(TW, KS, 4, P);  \
        else SCAN_LAUNCH_C(TW, KS, 2, P);           \
    } while (0)
#define SCAN_LAUNCH_T(TW, P)                                   \
    do {                                                       \
        if (per_thread <= 1) SCAN_LAUNCH(TW, 1, P);            \
        else if (per_thread <= 2) SCAN_LAUNCH(TW, 2, P);       \
        else if (per_thread <= 4) SCAN_LAUNCH(TW, 4, P);       \
        else if (per_thread <= 8) SCAN_LAUNCH(TW, 8, P);       \
        else if (per_thread <= 16) SCAN_LAUNCH(TW, 16, P);     \
        else if (per_thread <= 32) SCAN_LAUNCH(TW, 32, P);     \
        else SCAN_LAUNCH(TW, 64, P);                           \
    } while (0)
    if (w2 == nullptr)
        SCAN_LAUNCH_T(float, false);
    else if (w2_dtype == JK_BF16)
        SCAN_LAUNCH_T(__nv_bfloat16, true);
    else
        SCAN_LAUNCH_T(float, true);
    JK_CHECK_LAUNCH("linear_scan");
    if (n_pieces > 0) {
        jk_launch(scan_carry_kernel, dim3((dk * dv + 255) / 256, heads, n_piece_reqs), dim3(256), 0, stream, a);
        JK_CHECK_LAUNCH("scan_carry");
        if (dv <= 64) {
            const size_t pfx = pfx_smem(64, dk);
            if (pfx > 48 * 1024) cudaFuncSetAttribute(scan_prefix_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pfx);
            jk_launch(scan_prefix_kernel<64>, dim3(n_pieces, heads, 1), dim3(128), pfx, stream, a);
        } else {
            const size_t pfx = pfx_smem(PFX_COLS, dk);
            if (pfx > 48 * 1024) cudaFuncSetAttribute(scan_prefix_kernel<PFX_COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pfx);
            jk_launch(scan_prefix_kernel<PFX_COLS>, dim3(n_pieces, heads, (dv + PFX_COLS - 1) / PFX_COLS), dim3(128), pfx, stream, a);
        }
        JK_CHECK_LAUNCH("scan_prefix");
    }
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// What follows a linear attention: RMS norm of its output (over all heads' values at once with a weight of that size,
// or head by head with one weight of dv shared by the heads), times act(gate), into the activation type.
//     out[t, c] = o[t, c] / sqrt(mean_scope(o^2) + eps) * w[c or c % dv] * act(u[t, g_off + c])
// One block per row; a warp per head in the per-head forms (per_head 1: one weight of dv shared by the heads; 2: the mean
// per head, a weight of heads * dv).
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void norm_gate_kernel(const float *__restrict__ o, const float *__restrict__ u, int ld, int g_off, const float *__restrict__ w,
                                 float eps, int heads, int dv, int per_head, int gate_act, T *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x, n = heads * dv;
    const float *orow = o + (size_t)t * n;
    const float *grow = u + (size_t)t * ld + g_off;
    T *dst = out + (size_t)t * n;
    if (per_head) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
        for (int h = warp; h < heads; h += nwarp) {
            float ss = 0.f;
            for (int e = lane; e < dv; e += 32) { const float x = orow[h * dv + e]; ss += x * x; }
            const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dv + eps);
            for (int e = lane; e < dv; e += 32)
                dst[h * dv + e] = from_f32<T>(orow[h * dv + e] * inv * w[per_head == 2 ? h * dv + e : e] * apply_act(gate_act, grow[h * dv + e]));
        }
    } else {
        float ss = 0.f;
        for (int c = threadIdx.x; c < n; c += blockDim.x) { const float x = orow[c]; ss += x * x; }
        const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
        for (int c = threadIdx.x; c < n; c += blockDim.x) dst[c] = from_f32<T>(orow[c] * inv * w[c] * apply_act(gate_act, grow[c]));
    }
}

JK_EXPORT int jk_norm_gate(const float *o, const float *u, int ld, int g_off, const float *w, float eps, int heads, int dv,
                           int per_head, int gate_act, void *out, int dtype, int T, cudaStream_t stream) {
    if (T == 0) return JK_OK;
    JK_REQUIRE(o && u && w && out && heads > 0 && dv > 0, "norm_gate: an argument is missing");
    const int n = heads * dv;
    const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
    if (dtype == JK_F32)
        jk_launch(norm_gate_kernel<float>, dim3(T), dim3(threads), 0, stream, o, u, ld, g_off, w, eps, heads, dv, per_head, gate_act, (float *)out);
    else if (dtype == JK_BF16)
        jk_launch(norm_gate_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, o, u, ld, g_off, w, eps, heads, dv, per_head, gate_act,
                  (__nv_bfloat16 *)out);
    else
        JK_FAIL(JK_UNSUPPORTED, "norm_gate: dtype %d", dtype);
    JK_CHECK_LAUNCH("norm_gate");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Token shift: every projection of a mixer reads its own mixture of a row and the row before it in the sequence,
//     out[s, t] = T(h_t + (h_(t-1) - h_t) * mu[s])          s < parts, mu [parts, n] float32
// The row before a portion's first row is the request's last row of the step before, kept in last[slot, n] (zeros at the
// start of a sequence).  One block per row; `shift_last_kernel` then leaves each request's last row of this step in its
// slot; it runs after this kernel has read the slots.
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void token_shift_kernel(const T *__restrict__ h, const float *__restrict__ mu, const float *__restrict__ last,
                                   const int *__restrict__ row_req, const int *__restrict__ req_start, const int *__restrict__ slot_ids,
                                   T *__restrict__ out, int n, int parts, size_t part_stride, int vec) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int req = row_req[t];
    const bool first = t == req_start[req];
    const T *row = h + (size_t)t * n;
    const T *before = first ? nullptr : row - n;
    const float *kept = last + (size_t)slot_ids[req] * n;
    if (vec) {          // sixteen bytes of a row at a time (n a multiple of their elements, every base aligned)
        constexpr int E = 16 / sizeof(T);
        for (int c = threadIdx.x * E; c < n; c += blockDim.x * E) {
            float x[E], d[E];
            const uint4 xr = *reinterpret_cast<const uint4 *>(row + c);
            const T *xe = reinterpret_cast<const T *>(&xr);
            if (first) {
#pragma unroll
                for (int e = 0; e < E; e += 4) {
                    const float4 k4 = *reinterpret_cast<const float4 *>(kept + c + e);
                    d[e] = k4.x; d[e + 1] = k4.y; d[e + 2] = k4.z; d[e + 3] = k4.w;
                }
            } else {
                const uint4 br = *reinterpret_cast<const uint4 *>(before + c);
                const T *be = reinterpret_cast<const T *>(&br);
#pragma unroll
                for (int e = 0; e < E; ++e) d[e] = to_f32(be[e]);
            }
#pragma unroll
            for (int e = 0; e < E; ++e) { x[e] = to_f32(xe[e]); d[e] -= x[e]; }
            for (int s = 0; s < parts; ++s) {
                const float *m = mu + (size_t)s * n + c;
                uint4 o;
                T *oe = reinterpret_cast<T *>(&o);
#pragma unroll
                for (int e = 0; e < E; e += 4) {
                    const float4 m4 = *reinterpret_cast<const float4 *>(m + e);
                    oe[e] = from_f32<T>(fmaf(d[e], m4.x, x[e]));
                    oe[e + 1] = from_f32<T>(fmaf(d[e + 1], m4.y, x[e + 1]));
                    oe[e + 2] = from_f32<T>(fmaf(d[e + 2], m4.z, x[e + 2]));
                    oe[e + 3] = from_f32<T>(fmaf(d[e + 3], m4.w, x[e + 3]));
                }
                *reinterpret_cast<uint4 *>(out + (size_t)s * part_stride + (size_t)t * n + c) = o;
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float x = to_f32(row[c]);
        const float d = (first ? kept[c] : to_f32(before[c])) - x;
        for (int s = 0; s < parts; ++s) out[(size_t)s * part_stride + (size_t)t * n + c] = from_f32<T>(fmaf(d, mu[(size_t)s * n + c], x));
    }
}

template <typename T>
__global__ void shift_last_kernel(const T *__restrict__ h, float *__restrict__ last, const int *__restrict__ req_start,
                                  const int *__restrict__ slot_ids, int n) {
    pdl_trigger();
    pdl_wait();
    const int req = blockIdx.x;
    const int end = req_start[req + 1];
    if (end <= req_start[req]) return;
    const T *row = h + (size_t)(end - 1) * n;
    float *kept = last + (size_t)slot_ids[req] * n;
    for (int c = threadIdx.x; c < n; c += blockDim.x) kept[c] = to_f32(row[c]);
}

// h [T, n] (type `dtype`) -> out [parts, T, n]; last [slots, n] float32 moves on to the requests' last rows.
JK_EXPORT int jk_token_shift(const void *h, const float *mu, float *last, const int *row_req, const int *req_start, const int *slot_ids,
                             void *out, int dtype, int T, int nreq, int n, int parts, cudaStream_t stream) {
    if (T == 0 || nreq == 0) return JK_OK;
    JK_REQUIRE(h && mu && last && row_req && req_start && slot_ids && out && n > 0 && parts > 0, "token_shift: an argument is missing");
    int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
    const size_t stride = (size_t)T * n;
    const int per16 = dtype == JK_F32 ? 4 : 8;
    const int vec = n % per16 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)mu % 16 == 0 && (uintptr_t)last % 16 == 0 &&
                    (stride * (dtype == JK_F32 ? 4 : 2)) % 16 == 0;
    if (vec) threads = std::max(32, std::min(threads, (n / per16 + 31) / 32 * 32));
    if (dtype == JK_F32) {
        jk_launch(token_shift_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float *)h, mu, (const float *)last, row_req, req_start,
                  slot_ids, (float *)out, n, parts, stride, vec);
        jk_launch(shift_last_kernel<float>, dim3(nreq), dim3(threads), 0, stream, (const float *)h, last, req_start, slot_ids, n);
    } else if (dtype == JK_BF16) {
        jk_launch(token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16 *)h, mu, (const float *)last, row_req,
                  req_start, slot_ids, (__nv_bfloat16 *)out, n, parts, stride, vec);
        jk_launch(shift_last_kernel<__nv_bfloat16>, dim3(nreq), dim3(threads), 0, stream, (const __nv_bfloat16 *)h, last, req_start, slot_ids, n);
    } else {
        JK_FAIL(JK_UNSUPPORTED, "token_shift: dtype %d", dtype);
    }
    JK_CHECK_LAUNCH("token_shift");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// An activation between two products of a feed-forward without a gate: out[t, c] = T(act(u[t, c])), u float32 rows `ld` apart.
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void act_rows_kernel(const float *__restrict__ u, int ld, T *__restrict__ out, int n, size_t total, int act, int vec) {
    pdl_trigger();
    pdl_wait();
    if (vec) {          // four neighbouring columns of a row at a time (n and ld multiples of four, both bases aligned)
        const size_t quads = total / 4;
        const int per_row = n / 4;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
            const size_t t = i / per_row;
            const int c = (int)(i - t * per_row) * 4;
            const float4 x = *reinterpret_cast<const float4 *>(u + t * ld + c);
            __align__(16) T o[4] = {from_f32<T>(apply_act(act, x.x)), from_f32<T>(apply_act(act, x.y)), from_f32<T>(apply_act(act, x.z)),
                      from_f32<T>(apply_act(act, x.w))};
            if (sizeof(T) == 2) *reinterpret_cast<uint2 *>(out + t * n + c) = *reinterpret_cast<const uint2 *>(o);
            else *reinterpret_cast<uint4 *>(out + t * n + c) = *reinterpret_cast<const uint4 *>(o);
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / n;
        const int c = (int)(i - t * n);
        out[i] = from_f32<T>(apply_act(act, u[t * ld + c]));
    }
}

JK_EXPORT int jk_act_rows(const float *u, int ld, void *out, int dtype, int T, int n, int act, cudaStream_t stream) {
    if (T == 0) return JK_OK;
    JK_REQUIRE(u && out && n > 0 && ld >= n, "act_rows: an argument is missing");
    const size_t total = (size_t)T * n;
    const int vec = n % 4 == 0 && ld % 4 == 0 && (uintptr_t)u % 16 == 0 && (uintptr_t)out % 16 == 0;
    const int blocks = (int)std::min<size_t>(((vec ? total / 4 : total) + 255) / 256, 148 * 16);
    if (dtype == JK_F32)
        jk_launch(act_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, u, ld, (float *)out, n, total, act, vec);
    else if (dtype == JK_BF16)
        jk_launch(act_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, u, ld, (__nv_bfloat16 *)out, n, total, act, vec);
    else
        JK_FAIL(JK_UNSUPPORTED, "act_rows: dtype %d", dtype);
    JK_CHECK_LAUNCH("act_rows");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// The gated delta rule: per request and head, over the request's rows in order,
//     S <- g_t S;   w_t = beta_t (v_t - S^T k_t);   S <- S + k_t w_t^T;   o_t = S^T q_t          S [dk, dv], float32
// so a row's read-out sees its own write.  q and k come as float32 rows `c` (after their convolutions and activations),
// one head per key/value group (query head h reads group h / (heads / groups)), and are made unit vectors,
// x / sqrt(sum(x^2) + unit_eps), q also times q_scale; v likewise from `c`, one head per query head.  The write strength
// beta_t = sigmoid(u[t, b_off + h]) and the decay g_t = exp(-exp(A_log[h]) softplus(u[t, a_off + h] + dt_bias[h])) are
// formed in float32 from the float32 projection rows `u`.  S lives in state[slot, h] between steps.
//
// Two kernels.  delta_prep (a block a row) does what does not depend on the state, once per row instead of once per block
// of the scan: the unit vectors of every group, laid out as the scan's lanes read them, and per head (g, beta, k . q).
// delta_scan: a block owns DR_COLS value columns of one (request, head); DR_LANES neighbouring lanes share a column and
// keep the key channels part, part + DR_LANES, ... of it in registers (NPER each).  The prepared rows arrive DR_ROWS at a
// time by 16-byte asynchronous copies into two buffers that take turns, each lane's channels in 16-byte pieces on banks of
// their own.  Both sums over a column's lanes that a row needs are taken from the state BEFORE the row's write, so they
// run side by side and a row costs one round of shuffles:
//     a = S^T k,  b = S^T q  (old S);   w = beta (v - g a);   o = g b + w (k . q);   S <- g S + k w^T
// which is the recurrence above with o = (g S + k w^T)^T q multiplied out.  Two rows share a round the same way: the sums of
// row t + 1 against the state after row t are those against the state before row t, times g_t, plus w_t (k_t . k_(t+1)) and
// w_t (k_t . q_(t+1)); delta_prep leaves those two products of neighbouring rows with row t + 1, and the state takes both
// rows' writes at once, S <- g_(t+1) g_t S + g_(t+1) k_t w_t^T + k_(t+1) w_(t+1)^T.
// ---------------------------------------------------------------------------------------------------------------
constexpr int DR_LANES = 8, DR_COLS = 16, DR_THREADS = DR_LANES * DR_COLS, DR_ROWS = 32;

struct DeltaArgs {
    const float *c;             // [T, ld_c]: q at q_off (groups * dk), k at k_off (groups * dk), v at v_off (heads * dv)
    int ld_c, q_off, k_off, v_off;
    const float *u;             // [T, ld_u]: the write strength's logit at b_off + h, the decay's at a_off + h
    int ld_u, b_off, a_off;
    const float *A_log, *dt_bias;       // [heads]
    int heads, groups, dk, dv;
    float q_scale, unit_eps;
    float *state;               // [slots, heads, dk, dv]
    const int *req_start, *slot_ids;
    float *out;                 // [T, heads * dv]
    float *prep;                // [T, groups, 2, DR_LANES * nper] unit k then q, channel i at (i % DR_LANES) * nper + i / DR_LANES;
    float *scal;                // [T, heads, 8]: g, beta, k . q, 0; then k_(t-1) . k_t, k_(t-1) . q_t (unit vectors; row t - 1 of the step), 0, 0
    int nper;
};

// floats of scratch that T rows need
JK_EXPORT long long jk_delta_rule_scratch_floats(int T, int heads, int groups, int dk) {
    const int per = (dk + DR_LANES - 1) / DR_LANES, nper = per <= 4 ? 4 : (per <= 8 ? 8 : (per <= 16 ? 16 : 32));
    return (long long)T * ((long long)groups * 2 * DR_LANES * nper + 8LL * heads);
}

__global__ void __launch_bounds__(128) delta_prep_kernel(DeltaArgs a) {
    pdl_trigger();
    pdl_wait();
    __shared__ float kq_s[64], kk_prev_s[64], kq_prev_s[64];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, KW = DR_LANES * a.nper;
    const float *row = a.c + (size_t)t * a.ld_c;
    for (int g0 = 0; g0 < a.groups; g0 += 64) {
        for (int grp = g0 + warp; grp < min(a.groups, g0 + 64); grp += 4) {
            const float *kr = row + a.k_off + (size_t)grp * a.dk, *qr = row + a.q_off + (size_t)grp * a.dk;
            float sk = 0.f, sq = 0.f, kq = 0.f, sp = 0.f, pk = 0.f, pq = 0.f;
            for (int i = lane; i < a.dk; i += 32) { sk = fmaf(kr[i], kr[i], sk); sq = fmaf(qr[i], qr[i], sq); kq = fmaf(kr[i], qr[i], kq); }
            if (t > 0) {        // the row before (of the same request whenever the scan pairs the two)
                const float *pr = kr - a.ld_c;
                for (int i = lane; i < a.dk; i += 32) { sp = fmaf(pr[i], pr[i], sp); pk = fmaf(pr[i], kr[i], pk); pq = fmaf(pr[i], qr[i], pq); }
            }
            sk = warp_sum(sk); sq = warp_sum(sq); kq = warp_sum(kq); sp = warp_sum(sp); pk = warp_sum(pk); pq = warp_sum(pq);
            const float ik = 1.f / sqrtf(sk + a.unit_eps), iq = a.q_scale / sqrtf(sq + a.unit_eps), ip = 1.f / sqrtf(sp + a.unit_eps);
            float *dst = a.prep + ((size_t)t * a.groups + grp) * 2 * KW;
            for (int i = lane; i < KW; i += 32) {
                const int at = (i % DR_LANES) * a.nper + i / DR_LANES;
                dst[at] = i < a.dk ? kr[i] * ik : 0.f;
                dst[KW + at] = i < a.dk ? qr[i] * iq : 0.f;
            }
            if (lane == 0) { kq_s[grp - g0] = kq * ik * iq; kk_prev_s[grp - g0] = pk * ip * ik; kq_prev_s[grp - g0] = pq * ip * iq; }
        }
        __syncthreads();
        const int per_group = a.heads / a.groups;
        for (int h = g0 * per_group + threadIdx.x; h < min(a.groups, g0 + 64) * per_group; h += blockDim.x) {
            const float *urow = a.u + (size_t)t * a.ld_u;
            const float z = urow[a.a_off + h] + a.dt_bias[h];
            const float sp = z > 20.f ? z : log1pf(expf(z));
            float4 v;
            v.x = expf(-expf(a.A_log[h]) * sp);
            v.y = sigmoid_f(urow[a.b_off + h]);
            v.z = kq_s[h / per_group - g0];
            v.w = 0.f;
            *reinterpret_cast<float4 *>(a.scal + ((size_t)t * a.heads + h) * 8) = v;
            *reinterpret_cast<float4 *>(a.scal + ((size_t)t * a.heads + h) * 8 + 4) = make_float4(kk_prev_s[h / per_group - g0], kq_prev_s[h / per_group - g0], 0.f, 0.f);
        }
        __syncthreads();
    }
}

__device__ __forceinline__ void dr_copy4(float *dst, const float *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_copy16(float *dst, const float *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int NPER>
__global__ void __launch_bounds__(DR_THREADS) delta_scan_kernel(DeltaArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int LP = NPER + 4, KP = DR_LANES * LP;        // a lane's channels, padded so that the lanes' pieces fall on different banks
    constexpr int ROWF = 2 * KP + DR_COLS + 8;              // floats a row takes in shared memory: k, q, the block's values, the row's eight numbers
    constexpr int KW = DR_LANES * NPER, PIECES = KW / 4;
    extern __shared__ __align__(16) float dr_smem[];        // [2][DR_ROWS][ROWF]
    const int h = blockIdx.x, req = blockIdx.y, col0 = blockIdx.z * DR_COLS;
    const int group = h / (a.heads / a.groups);
    const int part = threadIdx.x % DR_LANES, cl = threadIdx.x / DR_LANES, col = col0 + cl;
    const bool live = col < a.dv;
    const int first = a.req_start[req], n = a.req_start[req + 1] - first;
    float *S = a.state + (((size_t)a.slot_ids[req] * a.heads + h) * a.dk) * a.dv;
    const size_t voff = a.v_off + (size_t)h * a.dv + col0;
    auto fetch = [&](int r0, float *buf) {
        const int nr = min(DR_ROWS, n - r0);
        for (int i = threadIdx.x; i < nr * 2 * PIECES; i += DR_THREADS) {
            const int r = i / (2 * PIECES), p = i % (2 * PIECES), which = p / PIECES, pp = p % PIECES;
            const float *src = a.prep + ((size_t)(first + r0 + r) * a.groups + group) * 2 * KW + which * KW + pp * 4;
            dr_copy16(buf + r * ROWF + which * KP + (pp / (NPER / 4)) * LP + (pp % (NPER / 4)) * 4, src);
        }
        for (int i = threadIdx.x; i < nr * DR_COLS; i += DR_THREADS) {
            const int r = i / DR_COLS, cc = i % DR_COLS;
            if (col0 + cc < a.dv) dr_copy4(buf + r * ROWF + 2 * KP + cc, a.c + (size_t)(first + r0 + r) * a.ld_c + voff + cc);
        }
        if (threadIdx.x < 2 * nr)
            dr_copy16(buf + (threadIdx.x >> 1) * ROWF + 2 * KP + DR_COLS + 4 * (threadIdx.x & 1),
                      a.scal + ((size_t)(first + r0 + (threadIdx.x >> 1)) * a.heads + h) * 8 + 4 * (threadIdx.x & 1));
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    float s[NPER];
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
        const int i = part + DR_LANES * j;
        s[j] = (live && i < a.dk) ? S[(size_t)i * a.dv + col] : 0.f;
    }
    if (n > 0) fetch(0, dr_smem);
    int turn = 0;
    for (int r0 = 0; r0 < n; r0 += DR_ROWS, turn ^= 1) {
        const int nr = min(DR_ROWS, n - r0);
        const float *buf = dr_smem + turn * DR_ROWS * ROWF;
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();        // this chunk's rows are there, and everyone is done with the other buffer
        if (r0 + DR_ROWS < n) fetch(r0 + DR_ROWS, dr_smem + (turn ^ 1) * DR_ROWS * ROWF);
        float *orow = a.out + (size_t)(first + r0) * a.heads * a.dv + (size_t)h * a.dv + col;
        int r = 0;
        for (; r + 1 < nr; r += 2) {        // two rows a round
            const float *row1 = buf + r * ROWF, *row2 = row1 + ROWF;
            const float4 n1 = *reinterpret_cast<const float4 *>(row1 + 2 * KP + DR_COLS);       // g, beta, k . q
            const float4 n2 = *reinterpret_cast<const float4 *>(row2 + 2 * KP + DR_COLS);
            const float4 x2 = *reinterpret_cast<const float4 *>(row2 + 2 * KP + DR_COLS + 4);   // k1 . k2, k1 . q2
            const float v1 = live ? row1[2 * KP + cl] : 0.f, v2 = live ? row2[2 * KP + cl] : 0.f;
            float k1[NPER], k2[NPER];
            float a1 = 0.f, b1 = 0.f, a2 = 0.f, b2 = 0.f;
#pragma unroll
            for (int j = 0; j < NPER; j += 4) {
                const float4 ka = *reinterpret_cast<const float4 *>(row1 + part * LP + j), qa = *reinterpret_cast<const float4 *>(row1 + KP + part * LP + j);
                const float4 kb = *reinterpret_cast<const float4 *>(row2 + part * LP + j), qb = *reinterpret_cast<const float4 *>(row2 + KP + part * LP + j);
                k1[j] = ka.x; k1[j + 1] = ka.y; k1[j + 2] = ka.z; k1[j + 3] = ka.w;
                k2[j] = kb.x; k2[j + 1] = kb.y; k2[j + 2] = kb.z; k2[j + 3] = kb.w;
                a1 = fmaf(s[j], ka.x, a1); a1 = fmaf(s[j + 1], ka.y, a1); a1 = fmaf(s[j + 2], ka.z, a1); a1 = fmaf(s[j + 3], ka.w, a1);
                b1 = fmaf(s[j], qa.x, b1); b1 = fmaf(s[j + 1], qa.y, b1); b1 = fmaf(s[j + 2], qa.z, b1); b1 = fmaf(s[j + 3], qa.w, b1);
                a2 = fmaf(s[j], kb.x, a2); a2 = fmaf(s[j + 1], kb.y, a2); a2 = fmaf(s[j + 2], kb.z, a2); a2 = fmaf(s[j + 3], kb.w, a2);
                b2 = fmaf(s[j], qb.x, b2); b2 = fmaf(s[j + 1], qb.y, b2); b2 = fmaf(s[j + 2], qb.z, b2); b2 = fmaf(s[j + 3], qb.w, b2);
            }
#pragma unroll
            for (int o = 1; o < DR_LANES; o <<= 1) {
                a1 += __shfl_xor_sync(0xffffffffu, a1, o); b1 += __shfl_xor_sync(0xffffffffu, b1, o);
                a2 += __shfl_xor_sync(0xffffffffu, a2, o); b2 += __shfl_xor_sync(0xffffffffu, b2, o);
            }
            const float w1 = n1.y * (v1 - n1.x * a1);
            const float o1 = fmaf(w1, n1.z, n1.x * b1);
            a2 = fmaf(w1, x2.x, n1.x * a2);         // against the state after the first row
            b2 = fmaf(w1, x2.y, n1.x * b2);
            const float w2 = n2.y * (v2 - n2.x * a2);
            const float o2 = fmaf(w2, n2.z, n2.x * b2);
            const float c0 = n2.x * n1.x, c1 = n2.x * w1;
#pragma unroll
            for (int j = 0; j < NPER; ++j) s[j] = fmaf(k2[j], w2, fmaf(k1[j], c1, c0 * s[j]));
            if (part == 0 && live) {
                orow[(size_t)r * a.heads * a.dv] = o1;
                orow[(size_t)(r + 1) * a.heads * a.dv] = o2;
            }
        }
        for (; r < nr; ++r) {               // a chunk's last row where it has an odd number
            const float *rowp = buf + r * ROWF;
            const float4 row = *reinterpret_cast<const float4 *>(rowp + 2 * KP + DR_COLS);      // g, beta, k . q
            const float v = live ? rowp[2 * KP + cl] : 0.f;
            const float *kp = rowp + part * LP, *qp = rowp + KP + part * LP;
            float kk[NPER];
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int j = 0; j < NPER; j += 4) {
                const float4 k4 = *reinterpret_cast<const float4 *>(kp + j), q4 = *reinterpret_cast<const float4 *>(qp + j);
                kk[j] = k4.x; kk[j + 1] = k4.y; kk[j + 2] = k4.z; kk[j + 3] = k4.w;
                a0 = fmaf(s[j], k4.x, a0); a1 = fmaf(s[j + 1], k4.y, a1); a0 = fmaf(s[j + 2], k4.z, a0); a1 = fmaf(s[j + 3], k4.w, a1);
                b0 = fmaf(s[j], q4.x, b0); b1 = fmaf(s[j + 1], q4.y, b1); b0 = fmaf(s[j + 2], q4.z, b0); b1 = fmaf(s[j + 3], q4.w, b1);
            }
            float sk = a0 + a1, sq = b0 + b1;
            sk += __shfl_xor_sync(0xffffffffu, sk, 1); sq += __shfl_xor_sync(0xffffffffu, sq, 1);
            sk += __shfl_xor_sync(0xffffffffu, sk, 2); sq += __shfl_xor_sync(0xffffffffu, sq, 2);
            sk += __shfl_xor_sync(0xffffffffu, sk, 4); sq += __shfl_xor_sync(0xffffffffu, sq, 4);
            const float w = row.y * (v - row.x * sk);
#pragma unroll
            for (int j = 0; j < NPER; ++j) s[j] = fmaf(kk[j], w, row.x * s[j]);
            if (part == 0 && live) orow[(size_t)r * a.heads * a.dv] = fmaf(w, row.z, row.x * sq);
        }
    }
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
        const int i = part + DR_LANES * j;
        if (live && i < a.dk) S[(size_t)i * a.dv + col] = s[j];
    }
}

// `scratch`: jk_delta_rule_scratch_floats(T, ...) floats
JK_EXPORT int jk_delta_rule(const float *c, int ld_c, int q_off, int k_off, int v_off, const float *u, int ld_u, int b_off, int a_off,
                            const float *A_log, const float *dt_bias, int heads, int groups, int dk, int dv, float q_scale, float unit_eps,
                            float *state, const int *req_start, const int *slot_ids, int nreq, float *out, float *scratch, int T,
                            cudaStream_t stream) {
    if (nreq == 0 || T == 0) return JK_OK;
    JK_REQUIRE(c && u && A_log && dt_bias && state && req_start && slot_ids && out && scratch, "delta_rule: an argument is missing");
    JK_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0 && dk > 0 && dv > 0, "delta_rule: %d heads on %d groups, sizes %d and %d", heads, groups, dk, dv);
    JK_REQUIRE(dk <= 32 * DR_LANES, "delta_rule: key heads of %d exceed %d", dk, 32 * DR_LANES);
    JK_REQUIRE(nreq <= 65535 && (dv + DR_COLS - 1) / DR_COLS <= 65535, "delta_rule: %d requests exceed one launch", nreq);
    JK_REQUIRE((uintptr_t)scratch % 16 == 0, "delta_rule: the scratch does not start on a 16-byte boundary");
    const int per = (dk + DR_LANES - 1) / DR_LANES, nper = per <= 4 ? 4 : (per <= 8 ? 8 : (per <= 16 ? 16 : 32));
    DeltaArgs a{c, ld_c, q_off, k_off, v_off, u, ld_u, b_off, a_off, A_log, dt_bias, heads, groups, dk, dv, q_scale, unit_eps, state, req_start,
                slot_ids, out, scratch, scratch + (size_t)T * groups * 2 * DR_LANES * nper, nper};
    jk_launch(delta_prep_kernel, dim3(T), dim3(128), 0, stream, a);
    JK_CHECK_LAUNCH("delta_prep");
    const dim3 grid(heads, nreq, (dv + DR_COLS - 1) / DR_COLS);
#define LAUNCH(NPER)                                                                                                                         \
    do {                                                                                                                                     \
        const size_t smem = (size_t)2 * DR_ROWS * (2 * DR_LANES * (NPER + 4) + DR_COLS + 8) * sizeof(float);                                 \
        if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<NPER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
        jk_launch(delta_scan_kernel<NPER>, grid, dim3(DR_THREADS), smem, stream, a);                                                         \
    } while (0)
    if (nper == 4) LAUNCH(4); else if (nper == 8) LAUNCH(8); else if (nper == 16) LAUNCH(16); else LAUNCH(32);
#undef LAUNCH
    JK_CHECK_LAUNCH("delta_scan");
    return JK_OK;
}
