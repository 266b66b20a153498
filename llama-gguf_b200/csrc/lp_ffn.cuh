// lp_ffn.cuh — the norm-after-sum layer form and the feed-forward kinds beside relu^2: the gated tanh-GELU layer and the mixture of
// experts (router, top-k weights, expert activations).  Included by layerprog.cu inside its anonymous namespace.
#pragma once

// x <- (alpha x + y) / sqrt(mean((alpha x + y)^2) + eps) * w, kept in f32; xc receives the same row in the compute type (the
// sublayers of such a layer read x itself, so this copy is the next GEMM's operand).  w = null: x is only copied (the embedding);
// y = null: nothing is added.
template <typename OutT>
__global__ void lp_postnorm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, OutT* __restrict__ xc, int width,
                                   float alpha, float eps) {
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * width;
    OutT* cr = xc + (size_t)r * width;
    if (!w) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) cr[c] = from_f<OutT>(xr[c]);
        return;
    }
    const float* yr = y ? y + (size_t)r * width : nullptr;
    __shared__ float red[33];
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = yr ? fmaf(alpha, xr[c], yr[c]) : alpha * xr[c];
        xr[c] = v;
        ss += v * v;
    }
    ss = wsum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
        t = wsum(t);
        if (threadIdx.x == 0) red[32] = 1.0f / sqrtf(t / (float)width + eps);
    }
    __syncthreads();
    const float inv = red[32];
    for (int c = threadIdx.x; c < width; c += blockDim.x) {   // (a thread reads back its own writes)
        const float v = xr[c] * inv * w[c];
        xr[c] = v;
        cr[c] = from_f<OutT>(v);
    }
}

__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

// out[r][n] = gelu_tanh(P[r][n]) * P[r][ff + n]: the fused projection holds [gate | up]
template <typename OutT>
__global__ void lp_gated_gelu_kernel(const float* __restrict__ P, int ldp, OutT* __restrict__ out, int ff, int R) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * ff) return;
    const int r = (int)(i / ff), n = (int)(i - (size_t)r * ff);
    const float* p = P + (size_t)r * ldp;
    out[i] = from_f<OutT>(gelu_tanh_f(p[n]) * p[ff + n]);
}

// Router: one warp per row.  z = P[r][0 .. E) (f32 logits of the fused projection).  The `top` largest logits are taken one after
// the other (of equal logits the lower index first); their weights are the softmax over the chosen logits only.  wts[r][e] is the
// weight of expert e (0 when it is not chosen); sel[r][k] / selw[r][k] list the chosen experts in the order they were taken.
__global__ void lp_moe_route_kernel(const float* __restrict__ P, int ldp, int E, int top, float* __restrict__ wts, int* __restrict__ sel,
                                    float* __restrict__ selw, int R) {
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= R) return;
    const float* z = P + (size_t)r * ldp;
    float* w = wts + (size_t)r * E;
    for (int e = lane; e < E; e += 32) w[e] = 0.0f;
    __syncwarp();
    float zmax = 0.0f, sum = 0.0f;
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (w[e] == 0.0f && (v > best || (v == best && e < bi))) { best = v; bi = e; }   // (chosen experts carry a mark != 0)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (k == 0) zmax = best;
        const float p = expf(best - zmax);
        sum += p;
        if (lane == 0) {
            w[bi] = -1.0f - p;          // mark; turned into the weight below
            sel[(size_t)r * top + k] = bi;
            selw[(size_t)r * top + k] = p;
        }
        __syncwarp();
    }
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32)
        if (w[e] != 0.0f) w[e] = (-1.0f - w[e]) * inv;
    for (int k = lane; k < top; k += 32) selw[(size_t)r * top + k] *= inv;
}

// out[r][c] = relu(P[r][off + c])^2 * (weight of the expert that owns column c; 1 for the always-on expert's columns behind them)
template <typename OutT>
__global__ void lp_moe_act_kernel(const float* __restrict__ P, int ldp, int off, const float* __restrict__ wts, int E, int eff, int total,
                                  OutT* __restrict__ out, int R) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * total) return;
    const int r = (int)(i / total), c = (int)(i - (size_t)r * total);
    const int e = c / eff;
    const float wgt = e < E ? wts[(size_t)r * E + e] : 1.0f;
    float v = 0.0f;
    if (wgt != 0.0f) {
        const float z = fmaxf(P[(size_t)r * ldp + off + c], 0.0f);
        v = z * z * wgt;
    }
    out[i] = from_f<OutT>(v);
}
