// Kernels of blocks whose sublayers sit between two RMS norms, of attention over one small latent vector per token,
// of selective state-space scans and of routed experts:
//
//   norm_add            stream += rmsnorm(sublayer output) * w, and in the same pass the next sublayer's input
//                       rmsnorm(stream) * w'
//   concat_cast         [a | b] side by side as a product's operand; add_bias_rows
//   latent_qkv          queries split into their plain and rotated parts, the latent vector normed, the shared rotated
//                       key part turned, both written into the row's place of the paged cache
//   head_linear         one small product per head (the key and value maps of the latent attention moved to the
//                       query's and the output's side), optionally times a sigmoid gate
//   latent_attention    softmax attention of all heads over one cached row per position, whose leading elements are
//                       the values too; keys may be split among blocks (latent_merge joins them)
//   causal_conv         a short convolution over time per channel with bias and activation, and its tails
//   selective_scan      S <- exp(dt A) S + dt x B, y = S C + D x per channel, with dt = softplus(W low + b) formed here
//   route_topk, route_sort, expert products, expert_combine      experts chosen per token by their scores
//   softcap             cap * tanh(logits / cap)
//
// Everything that the design wants in float32 is float32 here: norms, angles, scores and softmax weights, routers, the
// scan's state, decays, step sizes and gates.  Products take operands of the activation type T (float or bfloat16) and
// accumulate in float32.  A step's rows are laid out request after request (req_start), continue at req_pos, and keep
// their state in slot slot_ids[request]; a whole prompt, a portion and a single token are one case.
#include "common.cuh"

#include <algorithm>
#include <cstdlib>

JK_DEFINE_ERROR_BUFFER(jk_blocks)

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

enum BlockAct : int { BACT_NONE = 0, BACT_SILU = 1, BACT_GELU_TANH = 2, BACT_SIGMOID = 3, BACT_RELU = 4, BACT_SWISH_CLAMP = 6 };
__device__ __forceinline__ float block_act(int act, float z) {
    switch (act) {
        case BACT_SILU: return silu_f(z);
        case BACT_GELU_TANH: return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        case BACT_SIGMOID: return sigmoid_f(z);
        case BACT_RELU: return fmaxf(z, 0.f);
        default: return z;
    }
}

// A gated unit's inner value from its two sums g and u and the score s of the row's choice (1 where the score multiplies the
// unit's output instead): act(s g) (s u), or, for BACT_SWISH_CLAMP, with g' = min(g, limit) and u' = clamp(u, -limit, limit),
// g' sigmoid(1.702 g') (u' + 1).
__device__ __forceinline__ float expert_inner(int act, float s, float g, float u, float limit) {
    if (act == BACT_SWISH_CLAMP) {
        g = fminf(s * g, limit);
        u = fminf(fmaxf(s * u, -limit), limit);
        return g * sigmoid_f(1.702f * g) * (u + 1.f);
    }
    return block_act(act, s * g) * (s * u);
}

#define BLOCKS_BY_DTYPE(dtype, name, LAUNCH)                                      \
    do {                                                                          \
        if ((dtype) == JK_F32) { LAUNCH(float); }                                 \
        else if ((dtype) == JK_BF16) { LAUNCH(__nv_bfloat16); }                   \
        else JK_FAIL(JK_UNSUPPORTED, name ": dtype %d", (int)(dtype));            \
    } while (0)

// ---------------------------------------------------------------------------------------------------------------
// x[r] += delta[r] / sqrt(mean(delta[r]^2) + eps) * w;  then, if `out` is given,
// out[r] = T(x[r] / sqrt(mean(x[r]^2) + eps2) * w_next)   (w_next null: out[r] = T(x[r])).
// One block per row; the row stays in shared memory between the passes.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void store4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16 *p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned *>(&lo); raw.y = *reinterpret_cast<const unsigned *>(&hi);
    *reinterpret_cast<uint2 *>(p) = raw;
}

// VEC: the width is a multiple of four and every operand starts on a 16-byte boundary: four elements move at a time
template <typename T, bool VEC>
__global__ void norm_add_kernel(const float *__restrict__ delta, float *__restrict__ x, const float *__restrict__ w, float eps,
                                const float *__restrict__ w_next, float eps2, T *__restrict__ out, int d) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * d;
    constexpr int S = VEC ? 4 : 1;
    float ss = 0.f;
    for (int c = threadIdx.x * S; c < d; c += blockDim.x * S) {
        if (VEC) {
            const float4 v = *reinterpret_cast<const float4 *>(delta + base + c);
            *reinterpret_cast<float4 *>(row_buf + c) = v;
            ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        } else {
            const float v = delta[base + c];
            row_buf[c] = v;
            ss += v * v;
        }
    }
    const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
    float ss2 = 0.f;
    for (int c = threadIdx.x * S; c < d; c += blockDim.x * S) {
        if (VEC) {
            const float4 xv = *reinterpret_cast<const float4 *>(x + base + c), wv = *reinterpret_cast<const float4 *>(w + c);
            const float4 dv = *reinterpret_cast<const float4 *>(row_buf + c);
            const float4 nx = make_float4(xv.x + dv.x * inv * wv.x, xv.y + dv.y * inv * wv.y, xv.z + dv.z * inv * wv.z, xv.w + dv.w * inv * wv.w);
            *reinterpret_cast<float4 *>(x + base + c) = nx;
            *reinterpret_cast<float4 *>(row_buf + c) = nx;
            ss2 += (nx.x * nx.x + nx.y * nx.y) + (nx.z * nx.z + nx.w * nx.w);
        } else {
            const float nx = x[base + c] + row_buf[c] * inv * w[c];
            x[base + c] = nx;
            row_buf[c] = nx;
            ss2 += nx * nx;
        }
    }
    if (out == nullptr) return;
    const float inv2 = w_next != nullptr ? 1.f / sqrtf(block_sum(ss2, scratch) / (float)d + eps2) : 1.f;
    for (int c = threadIdx.x * S; c < d; c += blockDim.x * S) {
        if (VEC) {
            const float4 v = *reinterpret_cast<const float4 *>(row_buf + c);
            const float4 wv = w_next != nullptr ? *reinterpret_cast<const float4 *>(w_next + c) : make_float4(1.f, 1.f, 1.f, 1.f);
            store4(out + base + c, w_next != nullptr ? make_float4(v.x * inv2 * wv.x, v.y * inv2 * wv.y, v.z * inv2 * wv.z, v.w * inv2 * wv.w) : v);
        } else {
            out[base + c] = from_f32<T>(w_next != nullptr ? row_buf[c] * inv2 * w_next[c] : row_buf[c]);
        }
    }
}

JK_EXPORT int jk_norm_add(const float *delta, float *x, const float *w, float eps, const float *w_next, float eps2, void *out,
                          int dtype, int rows, int d, cudaStream_t stream) {
    if (rows == 0) return JK_OK;
    JK_REQUIRE(delta && x && w && rows > 0 && d > 0, "norm_add: rows %d, width %d", rows, d);
    const size_t smem = (size_t)d * sizeof(float);
    JK_REQUIRE(smem <= 200 * 1024, "norm_add: width %d does not fit shared memory", d);
    const bool vec = d % 4 == 0 && (uintptr_t)delta % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                     (w_next == nullptr || (uintptr_t)w_next % 16 == 0) && (out == nullptr || (uintptr_t)out % 16 == 0);
    // a step of few rows has few blocks: then a thread takes one vector of the row, so that a pass is one round of loads
    int threads = d >= 4096 ? 512 : (d >= 1024 ? 256 : 128);
    if (rows <= 64 && vec) threads = std::min(1024, std::max(threads, (d / 4 + 31) / 32 * 32));
#define LAUNCH_V(T, V)                                                                                                              \
    do {                                                                                                                            \
        if (smem > 48 * 1024) cudaFuncSetAttribute(norm_add_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        jk_launch(norm_add_kernel<T, V>, dim3(rows), dim3(threads), smem, stream, delta, x, w, eps, w_next, eps2, (T *)out, d);   \
    } while (0)
#define LAUNCH(T) if (vec) LAUNCH_V(T, true); else LAUNCH_V(T, false)
    BLOCKS_BY_DTYPE(dtype, "norm_add", LAUNCH);
#undef LAUNCH
#undef LAUNCH_V
    JK_CHECK_LAUNCH("norm_add");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// out[t] = T([a[t] | b[t]]): two float32 streams side by side as the operand of one product.
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void concat_cast_kernel(const float *__restrict__ a, const float *__restrict__ b, T *__restrict__ out, int d, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / (2 * d);
        const int c = (int)(i % (2 * d));
        out[i] = from_f32<T>(c < d ? a[t * d + c] : b[t * d + c - d]);
    }
}

JK_EXPORT int jk_concat_cast(const float *a, const float *b, void *out, int dtype, int rows, int d, cudaStream_t stream) {
    if (rows == 0) return JK_OK;
    JK_REQUIRE(a && b && out && rows > 0 && d > 0, "concat_cast: rows %d, width %d", rows, d);
    const size_t total = (size_t)rows * 2 * d;
    const int blocks = (int)std::min<size_t>((total + 255) / 256, 148 * 16);
#define LAUNCH(T) jk_launch(concat_cast_kernel<T>, dim3(blocks), dim3(256), 0, stream, a, b, (T *)out, d, total)
    BLOCKS_BY_DTYPE(dtype, "concat_cast", LAUNCH);
#undef LAUNCH
    JK_CHECK_LAUNCH("concat_cast");
    return JK_OK;
}

__global__ void add_bias_rows_kernel(float *__restrict__ x, const float *__restrict__ bias, int d, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) x[i] += bias[i % d];
}

JK_EXPORT int jk_add_bias_rows(float *x, const float *bias, int rows, int d, cudaStream_t stream) {
    if (rows == 0) return JK_OK;
    JK_REQUIRE(x && bias && rows > 0 && d > 0, "add_bias_rows: rows %d, width %d", rows, d);
    const size_t total = (size_t)rows * d;
    const int blocks = (int)std::min<size_t>((total + 255) / 256, 148 * 16);
    jk_launch(add_bias_rows_kernel, dim3(blocks), dim3(256), 0, stream, x, bias, d, total);
    JK_CHECK_LAUNCH("add_bias_rows");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Queries and cache rows of the latent attention, from the float32 rows u [T, ld] of one fused product:
//   u[t, q_off + h (dn + dr) + e]      head h of the query: dn plain elements, then dr that are rotated
//   u[t, kv_off + e]                   e < R: the latent vector before its norm; then dr elements of the shared key part
// Rotation of the first `rot_dims` of the dr elements in pairs (2i, 2i+1) by p * freq[i], formed in float32, with cos and
// sin times `mag`.  Out: q_plain [T, H dn] (the operand of the per-head product that moves the key map to the query),
// the rotated parts into q_full [T, H, R + dr] behind the R elements which that product fills, and the cache row of the
// position, [latent * norm weight / rms | rotated key part], into pages [pages, page_size, R + dr].  One block per row.
// ---------------------------------------------------------------------------------------------------------------
struct LatentQkvArgs {
    const float *u;
    int ld, q_off, kv_off, H, dn, dr, R, rot_dims;
    const float *freq;
    float mag, eps;
    const float *norm_w;
    const int *positions, *row_req, *block_table;
    int max_blocks, page_size;
    void *q_plain, *q_full, *pages;
    const float *q_norm_w;      // with it: q_plain [T, q_rank] = rmsnorm(u[q_off .. q_off + q_rank)) * q_norm_w, the queries' own latent
    int q_rank;                 // vector (the heads' queries are then a product of it, made by the records that follow)
};

template <typename T>
__global__ void latent_qkv_kernel(LatentQkvArgs a) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float *u = a.u + (size_t)t * a.ld;
    const int pos = a.positions[t];
    const float fpos = (float)pos;
    const int dq = a.dn + a.dr, D = a.R + a.dr;
    // the latent vector's norm
    float ss = 0.f;
    for (int e = threadIdx.x; e < a.R; e += blockDim.x) {
        const float v = u[a.kv_off + e];
        ss += v * v;
    }
    const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)a.R + a.eps);
    const int page = a.block_table[(size_t)a.row_req[t] * a.max_blocks + pos / a.page_size];
    T *crow = (T *)a.pages + ((size_t)page * a.page_size + (size_t)(pos % a.page_size)) * D;
    for (int e = threadIdx.x; e < a.R; e += blockDim.x) crow[e] = from_f32<T>(u[a.kv_off + e] * inv * a.norm_w[e]);
    if (a.q_norm_w != nullptr) {
        float sq = 0.f;
        for (int e = threadIdx.x; e < a.q_rank; e += blockDim.x) {
            const float v = u[a.q_off + e];
            sq += v * v;
        }
        const float inv_q = 1.f / sqrtf(block_sum(sq, scratch) / (float)a.q_rank + a.eps);
        for (int e = threadIdx.x; e < a.q_rank; e += blockDim.x)
            ((T *)a.q_plain)[(size_t)t * a.q_rank + e] = from_f32<T>(u[a.q_off + e] * inv_q * a.q_norm_w[e]);
        return;
    }
    // rotated parts: the shared key part (head index H) and every head's query part
    for (int idx = threadIdx.x; idx < (a.H + 1) * a.dr; idx += blockDim.x) {
        const int h = idx / a.dr, e = idx % a.dr;
        const float *src = h == a.H ? u + a.kv_off + a.R : u + a.q_off + (size_t)h * dq + a.dn;
        float val = src[e];
        if (e < a.rot_dims) {
            float sn, cs;
            sincosf(fpos * a.freq[e >> 1], &sn, &cs);
            sn *= a.mag; cs *= a.mag;
            const float other = src[e ^ 1];
            val = (e & 1) ? fmaf(val, cs, other * sn) : fmaf(val, cs, -other * sn);
        }
        if (h == a.H) crow[a.R + e] = from_f32<T>(val);
        else ((T *)a.q_full)[((size_t)t * a.H + h) * D + a.R + e] = from_f32<T>(val);
    }
    for (int idx = threadIdx.x; idx < a.H * a.dn; idx += blockDim.x) {
        const int h = idx / a.dn, e = idx % a.dn;
        ((T *)a.q_plain)[(size_t)t * a.H * a.dn + idx] = from_f32<T>(u[a.q_off + (size_t)h * dq + e]);
    }
}

JK_EXPORT int jk_latent_qkv(const float *u, int ld, int q_off, int kv_off, int H, int dn, int dr, int R, int rot_dims, const float *freq,
                            float mag, const float *norm_w, float eps, const int *positions, const int *row_req, const int *block_table,
                            int max_blocks, int page_size, void *q_plain, void *q_full, void *pages, int dtype, int T,
                            const float *q_norm_w, int q_rank, cudaStream_t stream) {
    if (T == 0) return JK_OK;
    JK_REQUIRE(u && norm_w && positions && row_req && block_table && q_plain && (q_full || q_norm_w) && pages, "latent_qkv: an argument is missing");
    JK_REQUIRE(q_norm_w == nullptr || (q_rank > 0 && dr == 0), "latent_qkv: queries through a latent of %d elements beside a rotated part of %d", q_rank, dr);
    JK_REQUIRE(H > 0 && dn >= 0 && dr >= 0 && R > 0 && page_size > 0, "latent_qkv: heads %d, sizes %d + %d, latent %d", H, dn, dr, R);
    JK_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0 && (rot_dims == 0 || freq), "latent_qkv: rotation of %d of %d elements", rot_dims, dr);
    LatentQkvArgs a{u, ld, q_off, kv_off, H, dn, dr, R, rot_dims, freq, mag, eps, norm_w, positions, row_req, block_table,
                    max_blocks, page_size, q_plain, q_full, pages, q_norm_w, q_rank};
    const int work = q_norm_w ? std::max(q_rank, R) : H * (dn + dr);
    const int threads = work >= 2048 ? 512 : (work >= 512 ? 256 : 128);
#define LAUNCH(TT) jk_launch(latent_qkv_kernel<TT>, dim3(T), dim3(threads), 0, stream, a)
    BLOCKS_BY_DTYPE(dtype, "latent_qkv", LAUNCH);
#undef LAUNCH
    JK_CHECK_LAUNCH("latent_qkv");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Tiled products: C[M, N] = A[M, K] W[N, K]^T with float32 accumulation, operands of type T.  A block of 256 threads
// makes a tile of 64 x 64.  float operands: on the CUDA cores (FFMA in the order of K, a thread 4 x 4 of the tile, K
// through shared memory 16 at a time).  bfloat16 operands: on the tensor cores (mma.sync m16n8k16, a warp 16 x 32 of the
// tile, K through shared memory 32 at a time by asynchronous copies three tiles deep, fragments by ldmatrix).  Rows of A may be picked through an index (a_rows).
// With GLU a second weight tile W2 runs along and the epilogue sees both sums.  A thread holds 16 sums; tile_at() says
// where sum e lies in the tile.  Used per head (head_linear) and per expert (expert products), where the problem depends
// on the block.
// ---------------------------------------------------------------------------------------------------------------
constexpr int GT_M = 64, GT_N = 64, GT_K = 16;

template <typename T> struct OnTensorCores { static constexpr bool value = false; };
template <> struct OnTensorCores<__nv_bfloat16> { static constexpr bool value = true; };

template <typename T>
__device__ __forceinline__ void tile_at(int e, int *row, int *col) {
    if (OnTensorCores<T>::value) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        *row = (warp & 3) * 16 + (lane >> 2) + ((e & 2) ? 8 : 0);
        *col = (warp >> 2) * 32 + (e >> 2) * 8 + (lane & 3) * 2 + (e & 1);
    } else {
        *row = (threadIdx.x / 16) * 4 + e / 4;
        *col = (threadIdx.x % 16) * 4 + e % 4;
    }
}

template <bool GLU>
__device__ __forceinline__ void tile_product(const float *__restrict__ A, size_t lda, const int *__restrict__ a_rows, int M,
                                             const float *__restrict__ W, const float *__restrict__ W2, size_t ldw, int N, int K, int m0, int n0,
                                             float (&acc)[16], float (&acc2)[16]) {
    __shared__ float As[GT_K][GT_M + 4];
    __shared__ float Ws[GT_K][GT_N + 4];
    __shared__ float W2s[GLU ? GT_K : 1][GT_N + 4];
    const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
    const int lr = tid / 4, lk = (tid % 4) * 4;      // this thread loads row lr, k lk .. lk + 3 of each operand tile
    const int am = m0 + lr, wn = n0 + lr;
    const float *arow = am < M ? A + (size_t)(a_rows ? a_rows[am] : am) * lda : nullptr;
    const float *wrow = wn < N ? W + (size_t)wn * ldw : nullptr;
    const float *w2row = (GLU && wn < N) ? W2 + (size_t)wn * ldw : nullptr;
#pragma unroll
    for (int e = 0; e < 16; ++e) { acc[e] = 0.f; acc2[e] = 0.f; }
    for (int k0 = 0; k0 < K; k0 += GT_K) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            As[lk + i][lr] = (arow && k < K) ? arow[k] : 0.f;
            Ws[lk + i][lr] = (wrow && k < K) ? wrow[k] : 0.f;
            if (GLU) W2s[lk + i][lr] = (w2row && k < K) ? w2row[k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GT_K; ++k) {
            float av[4], wv[4], w2v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = As[k][ty * 4 + i]; wv[i] = Ws[k][tx * 4 + i]; if (GLU) w2v[i] = W2s[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i * 4 + j] = fmaf(av[i], wv[j], acc[i * 4 + j]);
                    if (GLU) acc2[i * 4 + j] = fmaf(av[i], w2v[j], acc2[i * 4 + j]);
                }
        }
        __syncthreads();
    }
}

__device__ __forceinline__ void ldmatrix_x4(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, const void *smem_row) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float *d, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int TC_K = 32, TC_LD = TC_K + 8;     // rows of 80 bytes: 16-byte aligned for ldmatrix, and eight of them hit distinct banks

// eight elements of a row from k on; zeros beyond K or where there is no row
__device__ __forceinline__ uint4 fetch8(const __nv_bfloat16 *row, int k, int K, bool vec) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row != nullptr) {
        if (vec && k + 8 <= K) {
            v = *reinterpret_cast<const uint4 *>(row + k);
        } else {
            __nv_bfloat16 t[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) t[i] = k + i < K ? row[k + i] : __float2bfloat16_rn(0.f);
            v = *reinterpret_cast<const uint4 *>(t);
        }
    }
    return v;
}

// eight elements of a row from k on into shared memory, zeros beyond K or where there is no row: an asynchronous 16-byte
// copy where rows are 16-byte aligned, else element by element
__device__ __forceinline__ void stage8(__nv_bfloat16 *dst, const __nv_bfloat16 *row, int k, int K, bool vec) {
    if (vec) {
        const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
        const int left = row != nullptr ? K - k : 0;
        const int bytes = left >= 8 ? 16 : (left > 0 ? 2 * left : 0);
        const __nv_bfloat16 *src = bytes > 0 ? row + k : dst;          // nothing is read when bytes is 0; the address only has to be one
        if (bytes > 0) asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
        else *reinterpret_cast<uint4 *>(dst) = make_uint4(0u, 0u, 0u, 0u);
    } else {
        *reinterpret_cast<uint4 *>(dst) = fetch8(row, k, K, false);
    }
}

constexpr int TC_STAGES = 3;        // tiles of K in flight: a block keeps 2 x 5 KB (or 3 x with GLU) a stage on its way

template <bool GLU>
__device__ __forceinline__ void tile_product(const __nv_bfloat16 *__restrict__ A, size_t lda, const int *__restrict__ a_rows, int M,
                                             const __nv_bfloat16 *__restrict__ W, const __nv_bfloat16 *__restrict__ W2, size_t ldw, int N, int K,
                                             int m0, int n0, float (&acc)[16], float (&acc2)[16]) {
    __shared__ __align__(16) __nv_bfloat16 As[TC_STAGES][GT_M * TC_LD];
    __shared__ __align__(16) __nv_bfloat16 Ws[TC_STAGES][GT_N * TC_LD];
    __shared__ __align__(16) __nv_bfloat16 W2s[GLU ? TC_STAGES : 1][GLU ? GT_N * TC_LD : 8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int lr = tid / 4, lk = (tid % 4) * 8;      // this thread stages row lr, k lk .. lk + 7 of each operand tile
    const int am = m0 + lr, wn = n0 + lr;
    const __nv_bfloat16 *arow = am < M ? A + (size_t)(a_rows ? a_rows[am] : am) * lda : nullptr;
    const __nv_bfloat16 *wrow = wn < N ? W + (size_t)wn * ldw : nullptr;
    const __nv_bfloat16 *w2row = (GLU && wn < N) ? W2 + (size_t)wn * ldw : nullptr;
    const bool vec_a = lda % 8 == 0 && (uintptr_t)A % 16 == 0;
    const bool vec_w = ldw % 8 == 0 && (uintptr_t)W % 16 == 0 && (!GLU || (uintptr_t)W2 % 16 == 0);
#pragma unroll
    for (int e = 0; e < 16; ++e) { acc[e] = 0.f; acc2[e] = 0.f; }
    const int a_row = (warp & 3) * 16 + (lane & 15), a_col = (lane >> 4) * 8;
    const int b_row = (warp >> 2) * 32 + (lane >> 4) * 8 + (lane & 7), b_col = ((lane >> 3) & 1) * 8;
    const int nk = (K + TC_K - 1) / TC_K;
    auto stage = [&](int kt) {          // tile kt of K into its buffer; a group is committed even when there is no such tile
        if (kt < nk) {
            const int b = kt % TC_STAGES, k = kt * TC_K + lk;
            stage8(As[b] + lr * TC_LD + lk, arow, k, K, vec_a);
            stage8(Ws[b] + lr * TC_LD + lk, wrow, k, K, vec_w);
            if (GLU) stage8(W2s[b] + lr * TC_LD + lk, w2row, k, K, vec_w);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
#pragma unroll
    for (int i = 0; i < TC_STAGES - 1; ++i) stage(i);
    for (int kt = 0; kt < nk; ++kt) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(TC_STAGES - 2) : "memory");       // tile kt has landed (for this thread)
        __syncthreads();                                                                  // ... and for all; the buffer of tile kt - 1 is free
        stage(kt + TC_STAGES - 1);
        const __nv_bfloat16 *as = As[kt % TC_STAGES], *ws = Ws[kt % TC_STAGES], *w2s = W2s[GLU ? kt % TC_STAGES : 0];
#pragma unroll
        for (int kk = 0; kk < TC_K; kk += 16) {
            unsigned a0, a1, a2, a3;
            ldmatrix_x4(a0, a1, a2, a3, as + a_row * TC_LD + kk + a_col);
#pragma unroll
            for (int p = 0; p < 2; ++p) {          // two tiles of eight columns at a time
                unsigned b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, ws + (b_row + p * 16) * TC_LD + kk + b_col);
                mma_bf16_16816(acc + (2 * p) * 4, a0, a1, a2, a3, b0, b1);
                mma_bf16_16816(acc + (2 * p + 1) * 4, a0, a1, a2, a3, b2, b3);
                if (GLU) {
                    ldmatrix_x4(b0, b1, b2, b3, w2s + (b_row + p * 16) * TC_LD + kk + b_col);
                    mma_bf16_16816(acc2 + (2 * p) * 4, a0, a1, a2, a3, b0, b1);
                    mma_bf16_16816(acc2 + (2 * p + 1) * 4, a0, a1, a2, a3, b2, b3);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();        // a second product of the same block may stage at once
}

// C = A W^T for a float32 A and a bfloat16 W on the tensor cores without rounding A: every element of A is cut into two
// bfloat16 halves (a = hi + lo, which keeps 16 bits of its mantissa) and both halves meet the same weights.
__device__ __forceinline__ void tile_product_split(const float *__restrict__ A, size_t lda, int M, const __nv_bfloat16 *__restrict__ W, size_t ldw,
                                                   int N, int K, int m0, int n0, float (&acc)[16]) {
    __shared__ __align__(16) __nv_bfloat16 Ah[GT_M * TC_LD];
    __shared__ __align__(16) __nv_bfloat16 Al[GT_M * TC_LD];
    __shared__ __align__(16) __nv_bfloat16 Ws[GT_N * TC_LD];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int lr = tid / 4, lk = (tid % 4) * 8;
    const int am = m0 + lr, wn = n0 + lr;
    const float *arow = am < M ? A + (size_t)am * lda : nullptr;
    const __nv_bfloat16 *wrow = wn < N ? W + (size_t)wn * ldw : nullptr;
    const bool vec_w = ldw % 8 == 0 && (uintptr_t)W % 16 == 0;
#pragma unroll
    for (int e = 0; e < 16; ++e) acc[e] = 0.f;
    const int a_row = (warp & 3) * 16 + (lane & 15), a_col = (lane >> 4) * 8;
    const int b_row = (warp >> 2) * 32 + (lane >> 4) * 8 + (lane & 7), b_col = ((lane >> 3) & 1) * 8;
    for (int k0 = 0; k0 < K; k0 += TC_K) {
        __nv_bfloat16 h8[8], l8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int k = k0 + lk + i;
            const float v = (arow && k < K) ? arow[k] : 0.f;
            h8[i] = __float2bfloat16_rn(v);
            l8[i] = __float2bfloat16_rn(v - __bfloat162float(h8[i]));
        }
        *reinterpret_cast<uint4 *>(Ah + lr * TC_LD + lk) = *reinterpret_cast<const uint4 *>(h8);
        *reinterpret_cast<uint4 *>(Al + lr * TC_LD + lk) = *reinterpret_cast<const uint4 *>(l8);
        *reinterpret_cast<uint4 *>(Ws + lr * TC_LD + lk) = fetch8(wrow, k0 + lk, K, vec_w);
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TC_K; kk += 16) {
            unsigned h0, h1, h2, h3, l0, l1, l2, l3;
            ldmatrix_x4(h0, h1, h2, h3, Ah + a_row * TC_LD + kk + a_col);
            ldmatrix_x4(l0, l1, l2, l3, Al + a_row * TC_LD + kk + a_col);
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                unsigned b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, Ws + (b_row + p * 16) * TC_LD + kk + b_col);
                mma_bf16_16816(acc + (2 * p) * 4, l0, l1, l2, l3, b0, b1);
                mma_bf16_16816(acc + (2 * p + 1) * 4, l0, l1, l2, l3, b2, b3);
                mma_bf16_16816(acc + (2 * p) * 4, h0, h1, h2, h3, b0, b1);
                mma_bf16_16816(acc + (2 * p + 1) * 4, h0, h1, h2, h3, b2, b3);
            }
        }
        __syncthreads();
    }
}

// out[t, h * out_hs + n] = T(sum_k in[t, h * K + k] * w[h, n, k]) (* sigmoid(gate[t * gate_ld + h * N + n]))
template <typename T>
__global__ void __launch_bounds__(256) head_linear_kernel(const T *__restrict__ in, const T *__restrict__ w, T *__restrict__ out, int rows, int H,
                                                          int N, int K, int out_hs, const float *__restrict__ gate, int gate_ld) {
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.z, m0 = blockIdx.x * GT_M, n0 = blockIdx.y * GT_N;
    float acc[16], unused[16];
    tile_product<false>(in + (size_t)h * K, (size_t)H * K, nullptr, rows, w + (size_t)h * N * K, (const T *)nullptr, (size_t)K, N, K, m0, n0, acc, unused);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        int r, c;
        tile_at<T>(e, &r, &c);
        const int t = m0 + r, n = n0 + c;
        if (t >= rows || n >= N) continue;
        float v = acc[e];
        if (gate != nullptr) v *= sigmoid_f(gate[(size_t)t * gate_ld + (size_t)h * N + n]);
        out[((size_t)t * H + h) * out_hs + n] = from_f32<T>(v);
    }
}

JK_EXPORT int jk_head_linear(const void *in, const void *w, void *out, int dtype, int rows, int H, int N, int K, int out_hs,
                             const float *gate, int gate_ld, cudaStream_t stream) {
    if (rows == 0) return JK_OK;
    JK_REQUIRE(in && w && out && rows > 0 && H > 0 && N > 0 && K > 0 && out_hs >= N, "head_linear: rows %d, heads %d, %d x %d into %d", rows, H, N, K, out_hs);
    JK_REQUIRE(H <= 65535, "head_linear: %d heads exceed one launch", H);
    dim3 grid((rows + GT_M - 1) / GT_M, (N + GT_N - 1) / GT_N, H);
#define LAUNCH(T) jk_launch(head_linear_kernel<T>, grid, dim3(256), 0, stream, (const T *)in, (const T *)w, (T *)out, rows, H, N, K, out_hs, gate, gate_ld)
    BLOCKS_BY_DTYPE(dtype, "head_linear", LAUNCH);
#undef LAUNCH
    JK_CHECK_LAUNCH("head_linear");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Attention of H heads over one cached row per position: row j of a request is [c_j (R) | r_j (dr)]; a query row of a
// head is [a (R) | b (dr)]; score = (a . c_j + b . r_j) * scale over j <= position; out = sum_j softmax_j c_j  [R].
// A block takes one query row and LA_WARPS heads; 32 cached rows at a time pass shared memory (read once for all the
// block's heads), a lane takes one of them for the scores and a slice of R for the weighted sum.  Scores, the running
// maximum, the weights and the sums are float32.  With `splits` > 1 the keys of a row are cut into that many ranges
// (blockIdx.z); a range leaves its unnormalised sum, maximum and normaliser in `part` and latent_merge joins them.
// ---------------------------------------------------------------------------------------------------------------
constexpr int LA_WARPS = 8;

struct LatentAttnArgs {
    const void *q, *pages;
    void *out;
    float *part;            // [T, H, splits, R + 2]
    const int *positions, *row_req, *block_table;
    int T, H, R, dr, page_size, max_blocks, splits;
    float scale;
    int window;             // the mask as one number (jk_mask_lo): 0 every earlier key, W > 0 the last W keys
};

template <typename T, int NS>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(LatentAttnArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float la_smem[];
    const int D = a.R + a.dr, DP = D + 1;
    float *qs = la_smem;                                  // [LA_WARPS][D]
    float *tile = la_smem + LA_WARPS * D;                 // [32][D + 1]
    __shared__ long long row_off[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.y, h = blockIdx.x * LA_WARPS + warp;
    const bool active = h < a.H;
    const int pos = a.positions[t];
    const int *bt = a.block_table + (size_t)a.row_req[t] * a.max_blocks;
    int lo = jk_mask_lo(pos, a.window), hi = pos + 1;
    if (a.splits > 1) {
        const int chunk = (((hi - lo + a.splits - 1) / a.splits) + 31) / 32 * 32;
        lo += blockIdx.z * chunk;
        hi = min(pos + 1, lo + chunk);
    }
    if (active) {
        const T *qrow = (const T *)a.q + ((size_t)t * a.H + h) * D;
        for (int e = lane; e < D; e += 32) qs[warp * D + e] = to_f32(qrow[e]);
    }
    float m = -INFINITY, l = 0.f;
    float acc[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) acc[i] = 0.f;
    const T *pages = (const T *)a.pages;
    for (int j0 = lo; j0 < hi; j0 += 32) {
        const int n = min(32, hi - j0);
        if (threadIdx.x < 32) {
            const int j = j0 + threadIdx.x;
            row_off[threadIdx.x] = threadIdx.x < n ? ((long long)bt[j / a.page_size] * a.page_size + (j % a.page_size)) * D : -1;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < n * D; idx += blockDim.x) {
            const int r = idx / D, e = idx % D;
            tile[r * DP + e] = to_f32(pages[row_off[r] + e]);
        }
        __syncthreads();
        if (active) {
            float s = -INFINITY;
            if (lane < n) {
                const float *kr = tile + lane * DP, *qr = qs + warp * D;
                float dot = 0.f;
                for (int e = 0; e < D; ++e) dot = fmaf(qr[e], kr[e], dot);
                s = dot * a.scale;
            }
            const float m_new = fmaxf(m, warp_max(s));
            const float p = lane < n ? expf(s - m_new) : 0.f;
            const float corr = expf(m - m_new);
            l = l * corr + warp_sum(p);
            m = m_new;
#pragma unroll
            for (int i = 0; i < NS; ++i) acc[i] *= corr;
            for (int jj = 0; jj < n; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const float *vr = tile + jj * DP;
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    const int e = lane + 32 * i;
                    if (e < a.R) acc[i] = fmaf(pj, vr[e], acc[i]);
                }
            }
        }
        __syncthreads();
    }
    if (!active) return;
    if (a.splits > 1) {
        float *p = a.part + (((size_t)t * a.H + h) * a.splits + blockIdx.z) * (a.R + 2);
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            const int e = lane + 32 * i;
            if (e < a.R) p[e] = acc[i];
        }
        if (lane == 0) { p[a.R] = m; p[a.R + 1] = l; }
        return;
    }
    T *orow = (T *)a.out + ((size_t)t * a.H + h) * a.R;
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int e = lane + 32 * i;
        if (e < a.R) orow[e] = from_f32<T>(acc[i] * inv);
    }
}

// one block per (row, head): the ranges' sums brought to one maximum and added in the order of the ranges.  The ranges'
// factors exp(m_s - M) / l are formed once by the first warp (a lane a range) and kept in shared memory; a thread then
// takes columns, with all ranges' loads of a column asked for before the sum starts.
constexpr int LM_THREADS = 128, LM_MAX_SPLITS = 64;

template <typename T>
__global__ void __launch_bounds__(LM_THREADS) latent_merge_kernel(const float *__restrict__ part, T *__restrict__ out, int rows_heads, int R, int splits) {
    pdl_trigger();
    pdl_wait();
    __shared__ float factor[LM_MAX_SPLITS];
    const int lane = threadIdx.x & 31, idx = blockIdx.x;
    const float *p = part + (size_t)idx * splits * (R + 2);
    if (threadIdx.x < 32) {
        float ms[LM_MAX_SPLITS / 32], ls[LM_MAX_SPLITS / 32];
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < LM_MAX_SPLITS / 32; ++i) {
            const int s = lane + 32 * i;
            ms[i] = s < splits ? p[(size_t)s * (R + 2) + R] : -INFINITY;
            ls[i] = s < splits ? p[(size_t)s * (R + 2) + R + 1] : 0.f;
            M = fmaxf(M, ms[i]);
        }
        M = warp_max(M);
        float l = 0.f;
#pragma unroll
        for (int i = 0; i < LM_MAX_SPLITS / 32; ++i) {
            ms[i] = ms[i] > -INFINITY ? expf(ms[i] - M) : 0.f;
            l += ls[i] * ms[i];
        }
        l = warp_sum(l);
        const float inv = 1.f / l;
#pragma unroll
        for (int i = 0; i < LM_MAX_SPLITS / 32; ++i) {
            const int s = lane + 32 * i;
            if (s < splits) factor[s] = ms[i] * inv;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < R; e += LM_THREADS) {
        float v = 0.f;
        int s = 0;
        for (; s + 8 <= splits; s += 8) {
            float t[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) t[i] = p[(size_t)(s + i) * (R + 2) + e];
#pragma unroll
            for (int i = 0; i < 8; ++i) v = fmaf(t[i], factor[s + i], v);
        }
        for (; s < splits; ++s) v = fmaf(p[(size_t)s * (R + 2) + e], factor[s], v);
        out[(size_t)idx * R + e] = from_f32<T>(v);
    }
}

// The same attention on the tensor cores (bfloat16, mma.sync m16n8k16 with float32 accumulation).  Since every head reads
// the same cached rows, (query row, head) pairs are the M side of the products: a block of eight warps takes 32 pairs of
// one request (RT rows x HT heads) and walks the request's cached rows 32 at a time through shared memory.  Warp (mw, nw)
// has pairs mw * 16 .. + 15; for the scores it takes the tile's keys nw * 8 .. + 7 over the whole row width, the four nw
// warps exchange scores through shared memory, every thread forms the softmax weights of its own fragment (float32; the
// maximum and the sum go around the four lanes that share a row), and for the weighted sum it owns the output columns
// nw * NT * 8 .. of all 32 keys, the cached tile serving as the value operand through ldmatrix.trans.  Tiles of cached
// rows arrive by asynchronous copies into two buffers that take turns.  Ranges as above.
constexpr int LT_PAIRS = 32, LT_KEYS = 32;

struct LatentTcArgs {
    const __nv_bfloat16 *q, *pages;
    __nv_bfloat16 *out;
    float *part;
    const int *positions, *req_start, *block_table;
    int nreq, H, R, dr, page_size, max_blocks, splits, HT, RT, ldk;
    float scale;
    int buffers;        // 2: the tile after the one at work is on its way; 1: where two would leave an SM room for one block only
    int window;         // the mask as one number (jk_mask_lo)
};

__device__ __forceinline__ void ldmatrix_x2(unsigned &r0, unsigned &r1, const void *smem_row) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, const void *smem_row) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned *>(&v);
}

template <int NT>       // tiles of eight output columns per warp
__global__ void __launch_bounds__(256) latent_attention_tc_kernel(LatentTcArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char lt_smem[];
    // the block's request and rows
    int req = -1, t0 = 0, nrows = 0;
    {
        int tiles = 0;
        for (int i = 0; i < a.nreq; ++i) {
            const int len = a.req_start[i + 1] - a.req_start[i];
            const int mine = (len + a.RT - 1) / a.RT;
            if ((int)blockIdx.x < tiles + mine) {
                const int local = ((int)blockIdx.x - tiles) * a.RT;
                req = i; t0 = a.req_start[i] + local; nrows = min(a.RT, len - local);
                break;
            }
            tiles += mine;
        }
    }
    if (req < 0) return;
    const int h0 = blockIdx.y * a.HT;
    const int D = a.R + a.dr, DP = (D + 15) / 16 * 16, LDK = a.ldk, LDQ = DP + 8;
    __nv_bfloat16 *Qs = reinterpret_cast<__nv_bfloat16 *>(lt_smem);                 // [32][LDQ]
    __nv_bfloat16 *Kbuf = Qs + LT_PAIRS * LDQ;                                      // two tiles of [32][LDK] that take turns
    float *Sb = reinterpret_cast<float *>(Kbuf + a.buffers * LT_KEYS * LDK);        // [2][16][33]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, mw = warp & 1, nw = warp >> 1;
    const bool vec = D % 8 == 0 && (uintptr_t)a.pages % 16 == 0 && (uintptr_t)a.q % 16 == 0;
    {
        const int q8 = LDQ / 8;
        for (int idx = tid; idx < LT_PAIRS * q8; idx += 256) {
            const int p = idx / q8, e = (idx % q8) * 8, r = p / a.HT, h = h0 + p % a.HT;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < nrows && h < a.H && e < D) {
                const __nv_bfloat16 *src = a.q + ((size_t)(t0 + r) * a.H + h) * D + e;
                if (vec && e + 8 <= D) {
                    v = *reinterpret_cast<const uint4 *>(src);
                } else {
                    __nv_bfloat16 tmp[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) tmp[i] = e + i < D ? src[i] : __float2bfloat16_rn(0.f);
                    v = *reinterpret_cast<const uint4 *>(tmp);
                }
            }
            *reinterpret_cast<uint4 *>(Qs + p * LDQ + e) = v;
        }
    }
    const int max_pos = a.positions[t0 + nrows - 1];
    int lo = jk_mask_lo(a.positions[t0], a.window), hi = max_pos + 1;       // positions rise along a request's rows
    if (a.splits > 1) {
        const int chunk = (((hi - lo + a.splits - 1) / a.splits) + 31) / 32 * 32;
        lo += blockIdx.z * chunk;
        hi = min(max_pos + 1, lo + chunk);
    }
    // this thread's two rows of its warp's 16 pairs
    const int pa = mw * 16 + (lane >> 2), pb = pa + 8;
    const int ra = pa / a.HT, rb = pb / a.HT, ha = h0 + pa % a.HT, hb = h0 + pb % a.HT;
    const bool va = ra < nrows && ha < a.H, vb = rb < nrows && hb < a.H;
    const int pos_a = va ? a.positions[t0 + ra] : -1, pos_b = vb ? a.positions[t0 + rb] : -1;
    const int lo_a = jk_mask_lo(pos_a, a.window), lo_b = jk_mask_lo(pos_b, a.window);
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    const int *bt = a.block_table + (size_t)req * a.max_blocks;
    // A tile of cached rows into one of the two buffers: 16-byte asynchronous copies (zeros where there is no row or no
    // column) when rows are multiples of 16 bytes, else element by element.  The tile after the one at work is always
    // on its way.
    auto fetch_tile = [&](int j0, __nv_bfloat16 *Ks) {
        const int n = min(LT_KEYS, hi - j0);
        const __nv_bfloat16 *src_row[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {           // a warp brings rows warp, warp + 8, ...; their places first, then the copies
            const int r = warp + 8 * i, j = r < n ? j0 + r : lo;
            src_row[i] = a.pages + ((size_t)bt[j / a.page_size] * a.page_size + (size_t)(j % a.page_size)) * D;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = warp + 8 * i;
            __nv_bfloat16 *dst_row = Ks + r * LDK;
            for (int c = lane * 8; c < LDK; c += 256) {
                const bool there = r < n && c < D;
                if (vec) {
                    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_row + c);
                    const int bytes = there ? 16 : 0;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src_row[i] + (there ? c : 0)), "r"(bytes) : "memory");
                } else {
                    __nv_bfloat16 tmp[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) tmp[e] = (there && c + e < D) ? src_row[i][c + e] : __float2bfloat16_rn(0.f);
                    *reinterpret_cast<uint4 *>(dst_row + c) = *reinterpret_cast<const uint4 *>(tmp);
                }
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    const bool two = a.buffers > 1;
    if (lo < hi && two) fetch_tile(lo, Kbuf);
    int turn = 0;
    for (int j0 = lo; j0 < hi; j0 += LT_KEYS, turn ^= (two ? 1 : 0)) {
        const int n = min(LT_KEYS, hi - j0);
        const __nv_bfloat16 *Ks = Kbuf + turn * LT_KEYS * LDK;
        if (!two) {
            fetch_tile(j0, Kbuf);
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        } else if (j0 + LT_KEYS < hi) {
            fetch_tile(j0 + LT_KEYS, Kbuf + (turn ^ 1) * LT_KEYS * LDK);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        // scores of this warp's pairs against the keys nw * 8 .. + 7
        float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};      // two chains of sums that take turns
        {
            const __nv_bfloat16 *qp = Qs + (mw * 16 + (lane & 15)) * LDQ + (lane >> 4) * 8;
            const __nv_bfloat16 *kp = Ks + (nw * 8 + (lane & 7)) * LDK + ((lane >> 3) & 1) * 8;
            int kk = 0;
            for (; kk + 32 <= DP; kk += 32) {
                unsigned a0, a1, a2, a3, b0, b1, c0, c1, c2, c3, d0, d1;
                ldmatrix_x4(a0, a1, a2, a3, qp + kk);
                ldmatrix_x2(b0, b1, kp + kk);
                ldmatrix_x4(c0, c1, c2, c3, qp + kk + 16);
                ldmatrix_x2(d0, d1, kp + kk + 16);
                mma_bf16_16816(s, a0, a1, a2, a3, b0, b1);
                mma_bf16_16816(s2, c0, c1, c2, c3, d0, d1);
            }
            if (kk < DP) {
                unsigned a0, a1, a2, a3, b0, b1;
                ldmatrix_x4(a0, a1, a2, a3, qp + kk);
                ldmatrix_x2(b0, b1, kp + kk);
                mma_bf16_16816(s, a0, a1, a2, a3, b0, b1);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] += s2[i];
        }
        {
            float *row_a = Sb + (mw * 16 + (lane >> 2)) * 33, *row_b = row_a + 8 * 33;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int k = nw * 8 + (lane & 3) * 2 + c, j = j0 + k;
                row_a[k] = (k < n && j <= pos_a && j >= lo_a) ? s[c] * a.scale : -INFINITY;
                row_b[k] = (k < n && j <= pos_b && j >= lo_b) ? s[2 + c] * a.scale : -INFINITY;
            }
        }
        __syncthreads();
        // softmax weights of this thread's fragment: keys (lane & 3) * 2 + {0, 1} + {0, 8, 16, 24} of its two rows
        float pa_[8], pb_[8];
        {
            const float *row_a = Sb + (mw * 16 + (lane >> 2)) * 33, *row_b = row_a + 8 * 33;
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int k = g * 8 + (lane & 3) * 2 + c;
                    pa_[g * 2 + c] = row_a[k]; pb_[g * 2 + c] = row_b[k];
                    mx_a = fmaxf(mx_a, pa_[g * 2 + c]); mx_b = fmaxf(mx_b, pb_[g * 2 + c]);
                }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const float corr_a = mn_a == -INFINITY ? 1.f : expf(m_a - mn_a), corr_b = mn_b == -INFINITY ? 1.f : expf(m_b - mn_b);
            float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                pa_[i] = mn_a == -INFINITY ? 0.f : expf(pa_[i] - mn_a);
                pb_[i] = mn_b == -INFINITY ? 0.f : expf(pb_[i] - mn_b);
                sum_a += pa_[i]; sum_b += pb_[i];
            }
            sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1); sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
            sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1); sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
            l_a = l_a * corr_a + sum_a; l_b = l_b * corr_b + sum_b;
            m_a = mn_a; m_b = mn_b;
#pragma unroll
            for (int i = 0; i < NT; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }
        }
        // weighted sum: keys 0 .. 15, then 16 .. 31; values = the cached rows' columns nw * NT * 8 ..
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            const unsigned a0 = pack_bf16(pa_[ks * 4 + 0], pa_[ks * 4 + 1]), a1 = pack_bf16(pb_[ks * 4 + 0], pb_[ks * 4 + 1]);
            const unsigned a2 = pack_bf16(pa_[ks * 4 + 2], pa_[ks * 4 + 3]), a3 = pack_bf16(pb_[ks * 4 + 2], pb_[ks * 4 + 3]);
#pragma unroll
            for (int i = 0; i < NT; i += 2) {
                unsigned b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, Ks + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (nw * NT + i) * 8 + (lane >> 4) * 8);
                mma_bf16_16816(o[i], a0, a1, a2, a3, b0, b1);
                mma_bf16_16816(o[i + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const bool valid = half ? vb : va;
        if (!valid) continue;
        const int t = t0 + (half ? rb : ra), h = half ? hb : ha;
        const float l = half ? l_b : l_a, m = half ? m_b : m_a;
        if (a.splits > 1) {
            float *p = a.part + (((size_t)t * a.H + h) * a.splits + blockIdx.z) * (a.R + 2);
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int col = (nw * NT + i) * 8 + (lane & 3) * 2 + c;
                    if (col < a.R) p[col] = o[i][half * 2 + c];
                }
            if (nw == 0 && (lane & 3) == 0) { p[a.R] = m; p[a.R + 1] = l; }
        } else {
            __nv_bfloat16 *orow = a.out + ((size_t)t * a.H + h) * a.R;
            const float inv = 1.f / l;
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int col = (nw * NT + i) * 8 + (lane & 3) * 2 + c;
                    if (col < a.R) orow[col] = __float2bfloat16_rn(o[i][half * 2 + c] * inv);
                }
        }
    }
}

static bool latent_tc_enabled() {
    static const bool on = [] { const char *e = std::getenv("JK_LATENT_NO_TC"); return !(e && e[0] == '1'); }();
    return on;
}

// floats of `part` that `splits` ranges of T rows need
JK_EXPORT long long jk_latent_attention_scratch(int T, int H, int R, int splits) {
    return splits > 1 ? (long long)T * H * splits * (R + 2) : 0;
}

// `req_start` [nreq + 1] (may be null): with it, bfloat16 rows go to the tensor-core kernel (latent sizes up to 512).
JK_EXPORT int jk_latent_attention(const void *q, const void *pages, void *out, float *part, int dtype, const int *positions,
                                  const int *row_req, const int *block_table, int max_blocks, int page_size, int T, int H, int R,
                                  int dr, float scale, int splits, const int *req_start, int nreq, int window, cudaStream_t stream) {
    if (T == 0) return JK_OK;
    JK_REQUIRE(window >= 0, "latent_attention: window %d", window);
    JK_REQUIRE(q && pages && out && positions && row_req && block_table, "latent_attention: an argument is missing");
    JK_REQUIRE(H > 0 && R > 0 && dr >= 0 && page_size > 0 && max_blocks > 0, "latent_attention: heads %d, latent %d + %d", H, R, dr);
    JK_REQUIRE(R <= 1024, "latent_attention: a latent size of %d exceeds 1024", R);
    JK_REQUIRE(T <= 65535, "latent_attention: %d rows exceed one launch (65535)", T);
    if (splits < 1) splits = 1;
    JK_REQUIRE(splits == 1 || part != nullptr, "latent_attention: split keys need room for their parts");
    JK_REQUIRE(splits <= LM_MAX_SPLITS, "latent_attention: %d ranges exceed %d", splits, LM_MAX_SPLITS);
    const int D = R + dr;
    if (dtype == JK_BF16 && req_start != nullptr && nreq > 0 && R <= 512 && latent_tc_enabled()) {
        int HT = 1;
        while (HT * 2 <= std::min(H, LT_PAIRS)) HT *= 2;
        const int RT = LT_PAIRS / HT, tiles8 = (R + 7) / 8, per = (tiles8 + 3) / 4;
        const int NT = per <= 2 ? 2 : (per <= 4 ? 4 : (per <= 8 ? 8 : 16));
        const int DP = (D + 15) / 16 * 16, ldk = std::max(DP, 4 * NT * 8) + 8;
        // two tile buffers unless that leaves an SM (about 227 KB, 1 KB a block reserved) room for one block where one buffer leaves
        // room for two and the launch has more blocks than SMs
        const size_t fixed = (size_t)LT_PAIRS * (DP + 8) * 2 + 2 * 16 * 33 * sizeof(float), tile = (size_t)LT_KEYS * ldk * 2;
        dim3 grid((T + RT - 1) / RT + nreq, (H + HT - 1) / HT, splits);
        static const int sms = [] { int n = 148, dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev); return n; }();
        const bool second_block_fits = fixed + 2 * tile > 112 * 1024 && fixed + tile <= 112 * 1024;
        const int buffers = (second_block_fits && (long long)((T + RT - 1) / RT) * grid.y * grid.z > sms) ? 1 : 2;
        LatentTcArgs ta{(const __nv_bfloat16 *)q, (const __nv_bfloat16 *)pages, (__nv_bfloat16 *)out, part, positions, req_start, block_table,
                        nreq, H, R, dr, page_size, max_blocks, splits, HT, RT, ldk, scale, buffers, window};
        const size_t smem_tc = fixed + buffers * tile;
        JK_REQUIRE(grid.y <= 65535, "latent_attention: %d heads", H);
#define LAUNCH_TC(NT_)                                                                                                                       \
    do {                                                                                                                                    \
        if (smem_tc > 48 * 1024) cudaFuncSetAttribute(latent_attention_tc_kernel<NT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_tc); \
        jk_launch(latent_attention_tc_kernel<NT_>, grid, dim3(256), smem_tc, stream, ta);                                                   \
    } while (0)
        if (NT == 2) LAUNCH_TC(2); else if (NT == 4) LAUNCH_TC(4); else if (NT == 8) LAUNCH_TC(8); else LAUNCH_TC(16);
#undef LAUNCH_TC
        JK_CHECK_LAUNCH("latent_attention_tc");
        if (splits > 1) {
            const int n = T * H;
            jk_launch(latent_merge_kernel<__nv_bfloat16>, dim3(n), dim3(LM_THREADS), 0, stream, (const float *)part, (__nv_bfloat16 *)out, n, R, splits);
            JK_CHECK_LAUNCH("latent_merge");
        }
        return JK_OK;
    }
    LatentAttnArgs a{q, pages, out, part, positions, row_req, block_table, T, H, R, dr, page_size, max_blocks, splits, scale, window};
    const size_t smem = ((size_t)LA_WARPS * D + 32 * (size_t)(D + 1)) * sizeof(float);
    JK_REQUIRE(smem <= 220 * 1024, "latent_attention: rows of %d elements do not fit shared memory", D);
    dim3 grid((H + LA_WARPS - 1) / LA_WARPS, T, splits);
#define LAUNCH_NS(TT, NS)                                                                                                                   \
    do {                                                                                                                                    \
        if (smem > 48 * 1024) cudaFuncSetAttribute(latent_attention_kernel<TT, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        jk_launch(latent_attention_kernel<TT, NS>, grid, dim3(LA_WARPS * 32), smem, stream, a);                                             \
    } while (0)
#define LAUNCH(TT)                                  \
    if (R <= 64) LAUNCH_NS(TT, 2);                  \
    else if (R <= 128) LAUNCH_NS(TT, 4);            \
    else if (R <= 256) LAUNCH_NS(TT, 8);            \
    else if (R <= 512) LAUNCH_NS(TT, 16);           \
    else LAUNCH_NS(TT, 32)
    BLOCKS_BY_DTYPE(dtype, "latent_attention", LAUNCH);
#undef LAUNCH
#undef LAUNCH_NS
    JK_CHECK_LAUNCH("latent_attention");
    if (splits > 1) {
        const int n = T * H;
#define LAUNCH(TT) jk_launch(latent_merge_kernel<TT>, dim3(n), dim3(LM_THREADS), 0, stream, (const float *)part, (TT *)out, n, R, splits)
        BLOCKS_BY_DTYPE(dtype, "latent_merge", LAUNCH);
#undef LAUNCH
        JK_CHECK_LAUNCH("latent_merge");
    }
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// A short causal convolution over time on each of C channels, with bias and activation:
//     y_t[c] = act(bias[c] + sum_j taps[c, j] * u_(t - J + 1 + j)[c])          zeros before the sequence starts
// u is a column range of float32 rows [T, ld].  The J - 1 rows before a portion come from the request's tail
// [slots, J - 1, C] (s = J - 2 the newest), which conv_tails then moves forward.  y goes out as float32 (what a
// recurrence reads) and in the activation type (what a product reads).
// ---------------------------------------------------------------------------------------------------------------
struct ConvArgs {
    const float *u;
    int ld, off, C, J, act;
    const float *taps, *bias;
    float *tail;
    const int *row_req, *req_start, *slot_ids;
    float *y32;
    void *yT;
};

template <typename T>
__global__ void causal_conv_kernel(ConvArgs a, int rows) {
    pdl_trigger();
    pdl_wait();
    const size_t total = (size_t)rows * a.C;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / a.C), c = (int)(i % a.C);
        const int req = a.row_req[t];
        const int back = t - a.req_start[req];
        const float *tail = a.J > 1 ? a.tail + (size_t)a.slot_ids[req] * (a.J - 1) * a.C : nullptr;
        float acc = a.bias ? a.bias[c] : 0.f;
        for (int j = 0; j < a.J; ++j) {
            const int d = a.J - 1 - j;          // rows back
            const float uv = d <= back ? a.u[(size_t)(t - d) * a.ld + a.off + c] : tail[(size_t)(a.J - 1 + back - d) * a.C + c];
            acc = fmaf(a.taps[(size_t)c * a.J + j], uv, acc);
        }
        const float y = block_act(a.act, acc);
        if (a.y32) a.y32[i] = y;
        if (a.yT) ((T *)a.yT)[i] = from_f32<T>(y);
    }
}

// tail[slot, s, c] <- the input J - 1 - s rows before the end of the request's sequence after this step; a thread owns
// (request, channel) and reads every old entry before it overwrites it
__global__ void conv_tails_kernel(ConvArgs a, int nreq) {
    pdl_trigger();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nreq * a.C) return;
    const int req = idx / a.C, c = idx % a.C;
    const int first = a.req_start[req], n = a.req_start[req + 1] - first;
    float *tail = a.tail + (size_t)a.slot_ids[req] * (a.J - 1) * a.C;
    for (int s = 0; s < a.J - 1; ++s) {
        const int off = n - (a.J - 1) + s;
        const float v = off >= 0 ? a.u[(size_t)(first + off) * a.ld + a.off + c] : tail[(size_t)(s + n) * a.C + c];
        tail[(size_t)s * a.C + c] = v;
    }
}

JK_EXPORT int jk_causal_conv(const float *u, int ld, int off, int C, const float *taps, const float *bias, int J, int act, float *tail,
                             const int *row_req, const int *req_start, const int *slot_ids, float *y32, void *yT, int dtype, int T,
                             int nreq, cudaStream_t stream) {
    if (T == 0) return JK_OK;
    JK_REQUIRE(u && taps && row_req && req_start && C > 0 && J >= 1 && (y32 || yT), "causal_conv: an argument is missing");
    JK_REQUIRE(J == 1 || (tail && slot_ids), "causal_conv: %d taps without the tails' state", J);
    ConvArgs a{u, ld, off, C, J, act, taps, bias, tail, row_req, req_start, slot_ids, y32, yT};
    const size_t total = (size_t)T * C;
    const int blocks = (int)std::min<size_t>((total + 255) / 256, 148 * 16);
#define LAUNCH(TT) jk_launch(causal_conv_kernel<TT>, dim3(blocks), dim3(256), 0, stream, a, T)
    BLOCKS_BY_DTYPE(dtype, "causal_conv", LAUNCH);
#undef LAUNCH
    JK_CHECK_LAUNCH("causal_conv");
    if (J > 1) {
        jk_launch(conv_tails_kernel, dim3((nreq * C + 127) / 128), dim3(128), 0, stream, a, nreq);
        JK_CHECK_LAUNCH("conv_tails");
    }
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Selective scan.  Per request, channel c of E and state n of N, over the request's rows in order:
//     dt_t[c]  = softplus(sum_k Wdt[c, k] low_t[k] + bdt[c])                low_t = [dt part (K) | B_t (N) | C_t (N)]
//     S[c, n] <- exp(dt_t[c] A[c, n]) S[c, n] + dt_t[c] x_t[c] B_t[n]
//     y_t[c]   = sum_n S[c, n] C_t[n] + Dskip[c] x_t[c];   out_t[c] = T(y_t[c] * silu(z_t[c]))
// all float32; S lives in state[slot, c, n] between steps.  Eight neighbouring lanes share a channel: lane `part` keeps
// the states part, part + 8, ... in registers.  A block of 128 threads owns 16 channels of one request and walks the
// request's rows.
// ---------------------------------------------------------------------------------------------------------------
constexpr int SS_LANES = 8, SS_THREADS = 128, SS_CHANNELS = SS_THREADS / SS_LANES, SS_CHUNK = 32;

struct ScanArgs {
    const float *x;         // [T, E] after convolution and activation
    const float *low;       // [T, ld_low]
    int ld_low, K, N, E;
    const float *z;         // z_t[c] = z[t * ld_z + c]
    int ld_z;
    const void *Wdt;        // [E, K] in the activation type (float32 mode: float; bfloat16 mode: as the checkpoint stores it)
    const float *bdt, *A, *Dskip;
    float *state;
    const int *req_start, *slot_ids;
    void *out;
    const float *dt;        // step sizes made ahead, dt[t * ld_dt + c], or null: they are formed while the rows are staged
    int ld_dt;
};

// dt[t, c] = softplus(low[t, :K] . Wdt[c] + bdt[c]) ahead of the scan, as one product: float32 weights on the CUDA
// cores; bfloat16 weights (as a 16-bit checkpoint stores them) on the tensor cores with the float32 rows cut in two
// halves, so that nothing of them is rounded away.  The sums and the softplus are float32.
template <typename TW>
__global__ void __launch_bounds__(256) scan_steps_kernel(const float *__restrict__ low, int ld_low, const TW *__restrict__ Wdt,
                                                         const float *__restrict__ bdt, float *__restrict__ dt, int ld_dt, int rows, int E, int K) {
    pdl_trigger();
    pdl_wait();
    const int m0 = blockIdx.x * GT_M, n0 = blockIdx.y * GT_N;
    float acc[16];
    if constexpr (OnTensorCores<TW>::value) {
        tile_product_split(low, (size_t)ld_low, rows, Wdt, (size_t)K, E, K, m0, n0, acc);
    } else {
        float unused[16];
        tile_product<false>(low, (size_t)ld_low, nullptr, rows, Wdt, (const float *)nullptr, (size_t)K, E, K, m0, n0, acc, unused);
    }
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        int r, c;
        tile_at<TW>(e, &r, &c);
        const int t = m0 + r, ch = n0 + c;
        if (t < rows && ch < E) dt[(size_t)t * ld_dt + ch] = softplus_f(acc[e] + bdt[ch]);
    }
}

// Rows pass shared memory SS_CHUNK at a time (step sizes, inputs, B and C staged by all threads), so a row of the
// recurrence costs no global load and no exchange between lanes: a lane leaves its share of a row's sum in shared
// memory, and a chunk's outputs are added up and leave together, times silu(z).
template <typename T, int NPER>
__global__ void __launch_bounds__(SS_THREADS) selective_scan_kernel(ScanArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float ss_smem[];
    float *s_dt = ss_smem, *s_x = s_dt + SS_CHUNK * SS_CHANNELS, *s_y = s_x + SS_CHUNK * SS_CHANNELS;      // s_y: [chunk][threads]
    float *s_B = s_y + SS_CHUNK * SS_THREADS, *s_C = s_B + SS_CHUNK * a.N;
    const int req = blockIdx.y;
    const int part = threadIdx.x % SS_LANES, cl = threadIdx.x / SS_LANES;
    const int c0 = blockIdx.x * SS_CHANNELS, c = c0 + cl;
    const bool live = c < a.E;
    const int cc = live ? c : a.E - 1;          // idle lanes follow a real channel so that the shuffles stay whole
    const int first = a.req_start[req], last = a.req_start[req + 1];
    float *S = a.state + ((size_t)a.slot_ids[req] * a.E + cc) * a.N;
    float s[NPER], An[NPER];
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        const int n = part + SS_LANES * i;
        s[i] = n < a.N ? S[n] : 0.f;
        An[i] = n < a.N ? a.A[(size_t)cc * a.N + n] : 0.f;
    }
    for (int t0 = first; t0 < last; t0 += SS_CHUNK) {
        const int n_rows = min(SS_CHUNK, last - t0);
        // the loops below are unrolled so that a thread's loads are asked for together, not one after the other's arrival
#pragma unroll 4
        for (int idx = threadIdx.x; idx < SS_CHUNK * SS_CHANNELS; idx += SS_THREADS) {
            const int tt = idx / SS_CHANNELS, ch = min(c0 + idx % SS_CHANNELS, a.E - 1);
            if (tt >= n_rows) { s_dt[idx] = 0.f; s_x[idx] = 0.f; continue; }
            const size_t t = (size_t)(t0 + tt);
            float dt;
            if (a.dt != nullptr) {
                dt = a.dt[t * a.ld_dt + ch];
            } else {
                const float *low = a.low + t * a.ld_low;
                const T *w = (const T *)a.Wdt + (size_t)ch * a.K;
                float d = 0.f;
                for (int k = 0; k < a.K; ++k) d = fmaf(to_f32(w[k]), low[k], d);
                dt = softplus_f(d + a.bdt[ch]);
            }
            s_dt[idx] = dt;
            s_x[idx] = a.x[t * a.E + ch];
        }
#pragma unroll 4
        for (int idx = threadIdx.x; idx < SS_CHUNK * a.N; idx += SS_THREADS) {
            const int tt = idx / a.N, n = idx % a.N;
            const float *low = a.low + (size_t)(t0 + min(tt, n_rows - 1)) * a.ld_low + a.K;
            s_B[idx] = low[n];
            s_C[idx] = low[a.N + n];
        }
        __syncthreads();
        // four rows at a time: their step sizes, inputs, B and C into registers first, then the four updates in order, then
        // the four shares; rows beyond the chunk's end were staged as dt = 0, x = 0 and leave the state as it is
        for (int t4 = 0; t4 < n_rows; t4 += 4) {
            float dt4[4], dx4[4], B4[4][NPER], C4[4][NPER], y4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                dt4[j] = s_dt[(t4 + j) * SS_CHANNELS + cl];
                dx4[j] = dt4[j] * s_x[(t4 + j) * SS_CHANNELS + cl];
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    const int n = part + SS_LANES * i;
                    B4[j][i] = n < a.N ? s_B[(t4 + j) * a.N + n] : 0.f;
                    C4[j][i] = n < a.N ? s_C[(t4 + j) * a.N + n] : 0.f;
                }
            }
            float decay[4][NPER];
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < NPER; ++i) decay[j][i] = expf(dt4[j] * An[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float y = 0.f;
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    s[i] = fmaf(decay[j][i], s[i], dx4[j] * B4[j][i]);
                    y = fmaf(s[i], C4[j][i], y);
                }
                y4[j] = y;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) s_y[(t4 + j) * SS_THREADS + threadIdx.x] = y4[j];
        }
        __syncthreads();
#pragma unroll 4
        for (int idx = threadIdx.x; idx < n_rows * SS_CHANNELS; idx += SS_THREADS) {
            const int tt = idx / SS_CHANNELS, k = idx % SS_CHANNELS, ch = c0 + k;
            if (ch < a.E) {
                const size_t t = (size_t)(t0 + tt);
                const float *share = s_y + tt * SS_THREADS + k * SS_LANES;
                float y = 0.f;
#pragma unroll
                for (int i = 0; i < SS_LANES; ++i) y += share[i];
                y = fmaf(a.Dskip[ch], s_x[idx], y);
                ((T *)a.out)[t * a.E + ch] = from_f32<T>(y * silu_f(a.z[t * a.ld_z + ch]));
            }
        }
        __syncthreads();        // the next chunk's rows overwrite what this pass still reads
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
            const int n = part + SS_LANES * i;
            if (n < a.N) S[n] = s[i];
        }
    }
}

// `dt_buf` (may be null): room for step sizes [T, ld_dt], made ahead with one product; without it they are formed while
// the rows are staged.  `Wdt` is of the type `dtype` names.
JK_EXPORT int jk_selective_scan(const float *x, const float *low, int ld_low, int K, int N, int E, const float *z, int ld_z,
                                const void *Wdt, const float *bdt, const float *A, const float *Dskip, float *state,
                                const int *req_start, const int *slot_ids, int nreq, void *out, int dtype, float *dt_buf, int ld_dt,
                                int T, cudaStream_t stream) {
    if (nreq == 0) return JK_OK;
    JK_REQUIRE(x && low && z && Wdt && bdt && A && Dskip && state && req_start && slot_ids && out, "selective_scan: an argument is missing");
    JK_REQUIRE(K > 0 && N > 0 && E > 0 && ld_low >= K + 2 * N, "selective_scan: rank %d, states %d, channels %d, rows of %d", K, N, E, ld_low);
    JK_REQUIRE(N <= SS_LANES * 32, "selective_scan: %d states exceed %d", N, SS_LANES * 32);
    JK_REQUIRE(nreq <= 65535, "selective_scan: %d requests exceed one launch", nreq);
    const bool ahead = dt_buf != nullptr;
    if (ahead) {
        const dim3 tiles((T + GT_M - 1) / GT_M, (E + GT_N - 1) / GT_N);
#define LAUNCH(TT) jk_launch(scan_steps_kernel<TT>, tiles, dim3(256), 0, stream, low, ld_low, (const TT *)Wdt, bdt, dt_buf, ld_dt, T, E, K)
        BLOCKS_BY_DTYPE(dtype, "scan_steps", LAUNCH);
#undef LAUNCH
        JK_CHECK_LAUNCH("scan_steps");
    }
    ScanArgs a{x, low, ld_low, K, N, E, z, ld_z, Wdt, bdt, A, Dskip, state, req_start, slot_ids, out, ahead ? dt_buf : nullptr, ld_dt};
    dim3 grid((E + SS_CHANNELS - 1) / SS_CHANNELS, nreq);
    const int per = (N + SS_LANES - 1) / SS_LANES;
    const size_t smem = (size_t)SS_CHUNK * (2 * SS_CHANNELS + SS_THREADS + 2 * N) * sizeof(float);
#define LAUNCH_N(TT, NPER)                                                                                                                  \
    do {                                                                                                                                    \
        if (smem > 48 * 1024) cudaFuncSetAttribute(selective_scan_kernel<TT, NPER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        jk_launch(selective_scan_kernel<TT, NPER>, grid, dim3(SS_THREADS), smem, stream, a);                                                \
    } while (0)
#define LAUNCH(TT)                              \
    if (per <= 1) LAUNCH_N(TT, 1);              \
    else if (per <= 2) LAUNCH_N(TT, 2);         \
    else if (per <= 4) LAUNCH_N(TT, 4);         \
    else if (per <= 8) LAUNCH_N(TT, 8);         \
    else if (per <= 16) LAUNCH_N(TT, 16);       \
    else LAUNCH_N(TT, 32)
    BLOCKS_BY_DTYPE(dtype, "selective_scan", LAUNCH);
#undef LAUNCH
#undef LAUNCH_N
    JK_CHECK_LAUNCH("selective_scan");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Routed experts.  route_topk: one block per row; logits z_e = router[e] . h in float32, scores sigmoid(z_e); the `top`
// experts of largest score (the lower index wins a tie) -> ids, scores [T, top], and the experts' counts.  route_sort:
// one warp per expert lists its (row, choice) pairs in the order of the rows: entry -> source row, score; pair -> entry.
// The experts' products then run over the entries, expert after expert, as tiles of the grouped kernels below; an
// expert's input is score * h, which the first product applies to its sums (W (s h) = s (W h), in float32) before the
// gate's activation.  expert_combine adds a row's `top` results in the order of its choices.
// Options: a bias on the logits (`bias` [E]); a gate per row, sigmoid(gate_w . h), on what the sum is added to (a shared
// unit's output that waits in delta).
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void route_topk_kernel(const T *__restrict__ h, const float *__restrict__ router, int D, int E, int top, int *__restrict__ ids,
                                  float *__restrict__ scores, int *__restrict__ counts, int score_form, const float *__restrict__ bias,
                                  const float *__restrict__ gate_w, float *__restrict__ row_gate) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float z[];        // [E]
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const T *row = h + (size_t)t * D;
    const bool vec = D % 8 == 0 && (uintptr_t)row % 16 == 0 && (uintptr_t)router % 16 == 0;
    for (int e = warp; e < E; e += nwarp) {
        const float *w = router + (size_t)e * D;
        float dot = 0.f;
        if (vec) {          // eight elements a lane a pass, the passes' loads independent of one another
#pragma unroll 4
            for (int c = lane * 8; c < D; c += 256) {
                const float4 w0 = *reinterpret_cast<const float4 *>(w + c), w1 = *reinterpret_cast<const float4 *>(w + c + 4);
                float x[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = to_f32(row[c + i]);
                dot = fmaf(w0.x, x[0], dot); dot = fmaf(w0.y, x[1], dot); dot = fmaf(w0.z, x[2], dot); dot = fmaf(w0.w, x[3], dot);
                dot = fmaf(w1.x, x[4], dot); dot = fmaf(w1.y, x[5], dot); dot = fmaf(w1.z, x[6], dot); dot = fmaf(w1.w, x[7], dot);
            }
        } else {
            for (int c = lane; c < D; c += 32) dot = fmaf(w[c], to_f32(row[c]), dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) z[e] = dot + (bias ? bias[e] : 0.f);
    }
    if (gate_w != nullptr && warp == nwarp - 1) {       // the row's gate on what the experts' sum is added to: sigmoid(gate_w . h)
        float dot = 0.f;
        for (int c = lane; c < D; c += 32) dot = fmaf(gate_w[c], to_f32(row[c]), dot);
        dot = warp_sum(dot);
        if (lane == 0) row_gate[t] = sigmoid_f(dot);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // score_form 1: softmax over all experts; the chosen ones' scores divided by their sum
        float zmax = -INFINITY, total = 1.f, chosen = 0.f;
        if (score_form == 1) {
            for (int e = 0; e < E; ++e) zmax = fmaxf(zmax, z[e]);
            total = 0.f;
            for (int e = 0; e < E; ++e) total += expf(z[e] - zmax);
        }
        for (int k = 0; k < top; ++k) {
            int best = -1;
            float bz = -INFINITY;
            for (int e = 0; e < E; ++e)
                if (best < 0 || z[e] > bz) { bz = z[e]; best = e; }
            ids[(size_t)t * top + k] = best;
            const float sc = score_form == 1 ? expf(bz - zmax) / total : sigmoid_f(bz);
            scores[(size_t)t * top + k] = sc;
            chosen += sc;
            atomicAdd(&counts[best], 1);
            z[best] = -INFINITY;
        }
        if (score_form == 1)
            for (int k = 0; k < top; ++k) scores[(size_t)t * top + k] /= chosen + 1e-20f;
    }
}

// entry_row[pos], entry_score[pos] for pos in [starts[e], starts[e + 1]); pair_entry[pair] = pos
__global__ void route_sort_kernel(const int *__restrict__ ids, const float *__restrict__ scores, const int *__restrict__ counts, int pairs,
                                  int E, int top, int *__restrict__ starts, int *__restrict__ entry_row, float *__restrict__ entry_score,
                                  int *__restrict__ pair_entry) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (e >= E) return;
    int start = 0;
    for (int i = 0; i < e; ++i) start += counts[i];
    if (lane == 0) {
        starts[e] = start;
        if (e == E - 1) starts[E] = start + counts[e];
    }
    int at = start;
    for (int p0 = 0; p0 < pairs; p0 += 128) {          // four passes of 32 pairs, their loads asked for together
        int id[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int p = p0 + 32 * i + lane;
            id[i] = p < pairs ? ids[p] : -1;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int p = p0 + 32 * i + lane;
            const bool mine = id[i] == e;
            const unsigned ballot = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int pos = at + __popc(ballot & ((1u << lane) - 1u));
                entry_row[pos] = p / top;
                entry_score[pos] = scores[p];
                pair_entry[p] = pos;
            }
            at += __popc(ballot);
        }
    }
}

// which expert's tile a block has: tiles of GT_M entries, expert after expert
__device__ __forceinline__ bool expert_tile(const int *starts, int E, int block, int *expert, int *m0) {
    int tiles = 0;
    for (int e = 0; e < E; ++e) {
        const int n = starts[e + 1] - starts[e];
        const int mine = (n + GT_M - 1) / GT_M;
        if (block < tiles + mine) { *expert = e; *m0 = (block - tiles) * GT_M; return true; }
        tiles += mine;
    }
    return false;
}

// act[entry, n] = T(actf(s * g) * (s * u)), g = W_gate[e] h_row, u = W_up[e] h_row; w: [E, 2 ff, D] (gate rows, then up rows)
template <typename T>
__global__ void __launch_bounds__(256) expert_gate_up_kernel(const T *__restrict__ h, const T *__restrict__ w, T *__restrict__ act, int D, int ff, int E,
                                                             const int *__restrict__ starts, const int *__restrict__ entry_row,
                                                             const float *__restrict__ entry_score, int actf, float limit) {
    pdl_trigger();
    pdl_wait();
    int e, m0;
    if (!expert_tile(starts, E, blockIdx.x, &e, &m0)) return;
    const int first = starts[e], M = starts[e + 1] - first, n0 = blockIdx.y * GT_N;
    const T *we = w + (size_t)e * 2 * ff * D;
    float g[16], u[16];
    tile_product<true>(h, (size_t)D, entry_row + first, M, we, we + (size_t)ff * D, (size_t)D, ff, D, m0, n0, g, u);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        int r, c;
        tile_at<T>(e, &r, &c);
        r += m0;
        const int n = n0 + c;
        if (r >= M || n >= ff) continue;
        const float s = entry_score ? entry_score[first + r] : 1.f;
        act[(size_t)(first + r) * ff + n] = from_f32<T>(expert_inner(actf, s, g[e], u[e], limit));
    }
}

// y[entry, n] = W_down[e] act[entry]; w: [E, D, ff]; float32 out
template <typename T>
__global__ void __launch_bounds__(256) expert_down_kernel(const T *__restrict__ act, const T *__restrict__ w, float *__restrict__ y, int D, int ff, int E,
                                                          const int *__restrict__ starts) {
    pdl_trigger();
    pdl_wait();
    int e, m0;
    if (!expert_tile(starts, E, blockIdx.x, &e, &m0)) return;
    const int first = starts[e], M = starts[e + 1] - first, n0 = blockIdx.y * GT_N;
    float acc[16], unused[16];
    tile_product<false>(act + (size_t)first * ff, (size_t)ff, nullptr, M, w + (size_t)e * D * ff, (const T *)nullptr, (size_t)ff, D, ff, m0, n0, acc, unused);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        int r, c;
        tile_at<T>(i, &r, &c);
        r += m0;
        const int n = n0 + c;
        if (r < M && n < D) y[(size_t)(first + r) * D + n] = acc[i];
    }
}

// Steps of few rows (decoding): an expert has a handful of entries, and its matrices only have to stream past them.  A
// block of eight warps takes one expert and a slice of its output features; the expert's entries (up to ER_ROWS at a
// time) wait in shared memory; a warp takes one feature at a time, its lanes 16 bytes of the weight row each
// per pass, all loads of a row asked for before the sums start.  Float32 sums on the CUDA cores, in the order of K per
// lane and then across lanes, whatever else the step holds.
constexpr int ER_ROWS = 8, ER_FEATURES = 32;        // entries at a time; output features a block

template <typename T> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ void unpack16(const uint4 &v, float *f) {
    if constexpr (Vec16<T>::N == 4) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    } else {
        const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    }
}

// the features of one block against ROWS staged entries (the caller picks the smallest ROWS that holds them)
template <typename T, bool GLU, int ROWS>
__device__ __forceinline__ void expert_rows_features(const T *__restrict__ er_rows, const T *__restrict__ we, void *__restrict__ out, int K, int N,
                                                     int rows, size_t entry0, const float *__restrict__ entry_score, int actf, float limit) {
    constexpr int V = Vec16<T>::N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int f = warp; f < ER_FEATURES; f += 8) {
        const int n = blockIdx.y * ER_FEATURES + f;
        if (n >= N) break;
        const T *wg = we + (size_t)n * K, *wu = we + (size_t)(N + n) * K;
        float g[ROWS], u[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) { g[r] = 0.f; u[r] = 0.f; }
#pragma unroll 4
        for (int k = lane * V; k < K; k += 32 * V) {
            float a[V], b[V];
            unpack16<T>(*reinterpret_cast<const uint4 *>(wg + k), a);
            if (GLU) unpack16<T>(*reinterpret_cast<const uint4 *>(wu + k), b);
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                float x[V];
                unpack16<T>(*reinterpret_cast<const uint4 *>(er_rows + r * K + k), x);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    g[r] = fmaf(a[i], x[i], g[r]);
                    if (GLU) u[r] = fmaf(b[i], x[i], u[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            g[r] = warp_sum(g[r]);
            if (GLU) u[r] = warp_sum(u[r]);
        }
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (r >= rows) break;
                const size_t entry = entry0 + r;
                if (GLU) {
                    const float sc = entry_score ? entry_score[entry] : 1.f;
                    ((T *)out)[entry * N + n] = from_f32<T>(expert_inner(actf, sc, g[r], u[r], limit));
                } else {
                    ((float *)out)[entry * N + n] = g[r];
                }
            }
        }
    }
}

// GLU: act[entry, n] = T(actf(s g) (s u)) from rows of h picked by entry_row; else y[entry, n] = W[e][n] . in[entry]
template <typename T, bool GLU>
__global__ void __launch_bounds__(256) expert_rows_kernel(const T *__restrict__ in, const T *__restrict__ w, void *__restrict__ out, int K, int N, int E,
                                                          const int *__restrict__ starts, const int *__restrict__ entry_row,
                                                          const float *__restrict__ entry_score, int actf, float limit) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char er_smem[];
    T *er_rows = reinterpret_cast<T *>(er_smem);             // [ER_ROWS][K] as they are stored
    const int e = blockIdx.x, first = starts[e], M = starts[e + 1] - first;
    if (M <= 0) return;
    constexpr int V = Vec16<T>::N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T *we = w + (size_t)e * (GLU ? 2 : 1) * N * K;
    for (int r0 = 0; r0 < M; r0 += ER_ROWS) {
        const int rows = min(ER_ROWS, M - r0);
        __syncthreads();
        if (warp < rows) {      // warp r brings entry r: one look at where it lies, then 16 bytes a lane a pass
            const T *src = in + (size_t)(GLU ? entry_row[first + r0 + warp] : first + r0 + warp) * K;
#pragma unroll 4
            for (int k = lane * V; k < K; k += 32 * V)
                *reinterpret_cast<uint4 *>(er_rows + warp * K + k) = *reinterpret_cast<const uint4 *>(src + k);
        }
        __syncthreads();
        const size_t entry0 = (size_t)(first + r0);
        if (rows <= 1) expert_rows_features<T, GLU, 1>(er_rows, we, out, K, N, rows, entry0, entry_score, actf, limit);
        else if (rows <= 2) expert_rows_features<T, GLU, 2>(er_rows, we, out, K, N, rows, entry0, entry_score, actf, limit);
        else if (rows <= 4) expert_rows_features<T, GLU, 4>(er_rows, we, out, K, N, rows, entry0, entry_score, actf, limit);
        else expert_rows_features<T, GLU, 8>(er_rows, we, out, K, N, rows, entry0, entry_score, actf, limit);
    }
}

// delta[t] (+)= sum over the row's choices, in their order, of y[pair_entry[t * top + k]] (times the choice's score where
// `entry_score` is given: the form in which the score multiplies a unit's output)
__global__ void expert_combine_kernel(const float *__restrict__ y, const int *__restrict__ pair_entry, float *__restrict__ delta, int D, int top,
                                      int add, size_t total, const float *__restrict__ entry_score, const float *__restrict__ row_gate) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / D;
        const int c = (int)(i % D);
        float v = add ? (row_gate ? delta[i] * row_gate[t] : delta[i]) : 0.f;
        for (int k = 0; k < top; ++k) {
            const int entry = pair_entry[t * top + k];
            v = entry_score ? fmaf(entry_score[entry], y[(size_t)entry * D + c], v) : v + y[(size_t)entry * D + c];
        }
        delta[i] = v;
    }
}

// ints of workspace (`route`) that T rows need: counts [E], starts [E + 1], ids, entry_row, pair_entry [T top] and, as
// floats, scores and entry_score [T top] and the rows' gates [T]
JK_EXPORT long long jk_routed_experts_workspace(int T, int E, int top) { return 2LL * E + 1 + 5LL * T * top + T + 16; }

// h [T, D] (type T) -> delta [T, D] float32 (add: on top of what is there).  entries [T top, D]-sized buffers: `act`
// [T top, ff] of the activation type, `y` [T top, D] float32.
JK_EXPORT int jk_routed_experts(const void *h, const float *router, const void *w_gate_up, const void *w_down, float *delta, int add,
                                int dtype, int T, int D, int ff, int E, int top, int actf, int *route, void *act, float *y,
                                int score_form, float limit, const float *router_bias, const float *gate_w, cudaStream_t stream) {
    if (T == 0) return JK_OK;
    JK_REQUIRE(gate_w == nullptr || add, "routed_experts: a gate on a shared unit's output that is not there");
    JK_REQUIRE(h && router && w_gate_up && w_down && delta && route && act && y, "routed_experts: an argument is missing");
    JK_REQUIRE(D > 0 && ff > 0 && E > 0 && top > 0 && top <= E, "routed_experts: %d experts, %d a row, sizes %d and %d", E, top, D, ff);
    JK_REQUIRE((size_t)E * sizeof(float) <= 40 * 1024, "routed_experts: %d experts exceed the router's shared memory", E);
    const int pairs = T * top;
    int *counts = route, *starts = counts + E, *ids = starts + E + 1, *entry_row = ids + pairs, *pair_entry = entry_row + pairs;
    float *scores = (float *)(pair_entry + pairs), *entry_score = scores + pairs, *row_gate = gate_w ? entry_score + pairs : nullptr;
    if (cudaMemsetAsync(counts, 0, sizeof(int) * (size_t)E, stream) != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "routed_experts: clearing the counts failed");
#define LAUNCH(TT) jk_launch(route_topk_kernel<TT>, dim3(T), dim3(128), (size_t)E * sizeof(float), stream, (const TT *)h, router, D, E, top, ids, scores, counts, score_form, router_bias, gate_w, row_gate)
    BLOCKS_BY_DTYPE(dtype, "route_topk", LAUNCH);
#undef LAUNCH
    JK_CHECK_LAUNCH("route_topk");
    jk_launch(route_sort_kernel, dim3((E + 3) / 4), dim3(128), 0, stream, (const int *)ids, (const float *)scores, (const int *)counts, pairs, E, top,
              starts, entry_row, entry_score, pair_entry);
    JK_CHECK_LAUNCH("route_sort");
    // few rows: the experts' matrices stream past their entries (rows of 16-byte multiples); else tiles
    // score_form 1: the score multiplies the unit's output (in the sum of a row's choices), not its input
    const float *in_score = score_form == 1 ? nullptr : entry_score, *out_score = score_form == 1 ? entry_score : nullptr;
    const int per16 = dtype == JK_F32 ? 4 : 8;
    const bool stream_rows = pairs <= 64 && D % per16 == 0 && ff % per16 == 0 && (uintptr_t)w_gate_up % 16 == 0 && (uintptr_t)w_down % 16 == 0 &&
                             (size_t)ER_ROWS * std::max(D, ff) * 4 <= 160 * 1024;
    if (stream_rows) {
        const size_t elem = dtype == JK_F32 ? 4 : 2, smem_up = (size_t)ER_ROWS * D * elem, smem_down = (size_t)ER_ROWS * ff * elem;
#define LAUNCH(TT)                                                                                                                           \
    if (smem_up > 48 * 1024) cudaFuncSetAttribute(expert_rows_kernel<TT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up);  \
    if (smem_down > 48 * 1024) cudaFuncSetAttribute(expert_rows_kernel<TT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down); \
    jk_launch(expert_rows_kernel<TT, true>, dim3(E, (ff + ER_FEATURES - 1) / ER_FEATURES), dim3(256), smem_up, stream, (const TT *)h,        \
              (const TT *)w_gate_up, act, D, ff, E, (const int *)starts, (const int *)entry_row, in_score, actf, limit);          \
    jk_launch(expert_rows_kernel<TT, false>, dim3(E, (D + ER_FEATURES - 1) / ER_FEATURES), dim3(256), smem_down, stream, (const TT *)act,    \
              (const TT *)w_down, (void *)y, ff, D, E, (const int *)starts, (const int *)nullptr, (const float *)nullptr, 0, 0.f)
        BLOCKS_BY_DTYPE(dtype, "expert rows", LAUNCH);
#undef LAUNCH
        JK_CHECK_LAUNCH("expert rows");
    } else {
    const int tiles = (pairs + GT_M - 1) / GT_M + E;
#define LAUNCH(TT)                                                                                                                          \
    jk_launch(expert_gate_up_kernel<TT>, dim3(tiles, (ff + GT_N - 1) / GT_N), dim3(256), 0, stream, (const TT *)h, (const TT *)w_gate_up,  \
              (TT *)act, D, ff, E, (const int *)starts, (const int *)entry_row, in_score, actf, limit);                          \
    jk_launch(expert_down_kernel<TT>, dim3(tiles, (D + GT_N - 1) / GT_N), dim3(256), 0, stream, (const TT *)act, (const TT *)w_down, y, D, \
              ff, E, (const int *)starts)
    BLOCKS_BY_DTYPE(dtype, "expert products", LAUNCH);
#undef LAUNCH
    JK_CHECK_LAUNCH("expert products");
    }
    const size_t total = (size_t)T * D;
    jk_launch(expert_combine_kernel, dim3((int)std::min<size_t>((total + 255) / 256, 148 * 16)), dim3(256), 0, stream, (const float *)y,
              (const int *)pair_entry, delta, D, top, add, total, out_score, (const float *)row_gate);
    JK_CHECK_LAUNCH("expert_combine");
    return JK_OK;
}
// kernels that one call of jk_routed_experts launches (the clearing of the counts included)
JK_EXPORT int jk_routed_experts_launches() { return 6; }

// ---------------------------------------------------------------------------------------------------------------
// x[t] += table[index[t]] (index null: row `fixed` for every t): learned position vectors picked by the rows' positions,
// or one vector of a table added to the whole stream.  The table is float32 or of the compute type; the sum is float32.
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rows_kernel(float *__restrict__ x, const T *__restrict__ table, const int *__restrict__ index, int fixed, int d, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / d;
        const int row = index ? index[t] : fixed;
        x[i] += to_f32(table[(size_t)row * d + (i % d)]);
    }
}

JK_EXPORT int jk_add_rows(float *x, const void *table, int table_dtype, int table_rows, const int *index, int fixed, int rows, int d,
                          cudaStream_t stream) {
    if (rows == 0) return JK_OK;
    JK_REQUIRE(x && table && d > 0 && table_rows > 0 && (index || (fixed >= 0 && fixed < table_rows)), "add_rows: row %d of a table of %d", fixed, table_rows);
    const size_t total = (size_t)rows * d;
    const int blocks = (int)std::min<size_t>((total + 255) / 256, 148 * 16);
#define LAUNCH(TT) jk_launch(add_rows_kernel<TT>, dim3(blocks), dim3(256), 0, stream, x, (const TT *)table, index, fixed, d, total)
    BLOCKS_BY_DTYPE(table_dtype, "add_rows", LAUNCH);
#undef LAUNCH
    JK_CHECK_LAUNCH("add_rows");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// logits <- cap * tanh(logits / cap)
// ---------------------------------------------------------------------------------------------------------------
__global__ void softcap_kernel(float *__restrict__ x, float cap, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) x[i] = cap * tanhf(x[i] / cap);
}

JK_EXPORT int jk_softcap(float *x, float cap, long long n, cudaStream_t stream) {
    if (n == 0) return JK_OK;
    JK_REQUIRE(x && n > 0 && cap > 0.f, "softcap: %lld values, cap %f", n, (double)cap);
    jk_launch(softcap_kernel, dim3((int)std::min<long long>((n + 255) / 256, 148 * 16)), dim3(256), 0, stream, x, cap, (size_t)n);
    JK_CHECK_LAUNCH("softcap");
    return JK_OK;
}
