// A selective state-space mixer (state-space duality form with a scalar decay per head), token by
// token in float32:
//
//   xBC = silu(conv(xBC_in) + bias)            causal, per channel, `taps` wide, state = the last taps-1 inputs
//   dt  = softplus(dt_in + dt_bias),  a = exp(-exp(A_log) * dt)            per head
//   S_t = a S_(t-1) + dt B_t x_t^T            S: [N, P] per head, float32, carried per request
//   y_t = S_t^T C_t + D x_t
//   out = groupwise_rms(y * silu(z)) * w      in `groups` equal parts of the row
//
// Every request of the step brings its next tokens (one when it decodes, many in a prompt portion); its
// state lives in a slot of [slots, state_stride] floats: first the convolution's inputs [taps-1, C],
// then S as [heads, P, N].  The recurrence runs in the order of the tokens with a fixed order of sums, so
// what a position gets does not depend on how the prompt was cut or on the batch.
#include "common.cuh"

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ------------------------------------------------------------------ convolution + activation, dt and decay
// grid: (requests, channel blocks of 32 + 1).  The last block of a request turns dt_in into dt and the decay.
// Blocks of channels: 32 channels x 8 token lanes; each walks the request's tokens.
template <typename T>
__global__ void __launch_bounds__(256) ssm_conv_kernel(const T* __restrict__ zx, int ld, int c0, int C, int dt0, int H,
                                                       const float* __restrict__ cw, const float* __restrict__ cb, int taps,
                                                       const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                                       float* __restrict__ state, long long state_stride,
                                                       const int* __restrict__ cu_q, const int* __restrict__ slots,
                                                       float* __restrict__ xbc, float* __restrict__ dt_out,
                                                       float* __restrict__ decay_out) {
    const int s = blockIdx.x;
    const int slot = slots[s];
    const int q0 = cu_q[s], nq = cu_q[s + 1] - q0;
    if (slot < 0 || nq <= 0) return;
    const int cblocks = (C + 31) / 32;
    if ((int)blockIdx.y == cblocks) {
        for (int i = threadIdx.x; i < nq * H; i += blockDim.x) {
            const int t = i / H, h = i - t * H;
            const float dt = softplus_f(to_float(zx[(size_t)(q0 + t) * ld + dt0 + h]) + __ldg(dt_bias + h));
            dt_out[(size_t)(q0 + t) * H + h] = dt;
            decay_out[(size_t)(q0 + t) * H + h] = expf(-expf(__ldg(a_log + h)) * dt);
        }
        return;
    }
    const int lane_c = threadIdx.x & 31, lane_t = threadIdx.x >> 5;
    const int c = blockIdx.y * 32 + lane_c;
    const bool ok = c < C;
    float* st = state + (size_t)slot * state_stride;              // [taps-1][C]
    const int hist = taps - 1;
    if (ok) {
        const float bias = __ldg(cb + c);
        for (int t = lane_t; t < nq; t += 8) {
            float acc = bias;
            for (int k = 0; k < taps; ++k) {
                const int src = t - hist + k;
                const float v = src >= 0 ? to_float(zx[(size_t)(q0 + src) * ld + c0 + c]) : st[(size_t)(hist + src) * C + c];
                acc = fmaf(__ldg(cw + (size_t)c * taps + k), v, acc);
            }
            xbc[(size_t)(q0 + t) * C + c] = silu_f(acc);
        }
    }
    __syncthreads();                                                // every read of the old inputs is done
    if (ok && lane_t == 0) {
        // the last taps-1 inputs of [old inputs ; this step's inputs]; hist is small: a pass in place from the
        // front is safe, since entry j reads old entry j + nq >= j or a new input
        for (int j = 0; j < hist; ++j) {
            const int src = nq + j - hist;                          // index among this step's inputs
            st[(size_t)j * C + c] = src >= 0 ? to_float(zx[(size_t)(q0 + src) * ld + c0 + c]) : st[(size_t)(j + nq) * C + c];
        }
    }
}

PL_EXPORT int pl_ssm_conv(const void* zx, int dtype, int ld, int c0, int C, int dt0, int H, const float* cw, const float* cb,
                          int taps, const float* dt_bias, const float* a_log, float* state, long long state_stride,
                          const int* cu_q, const int* slots, int num_seqs, float* xbc, float* dt_out, float* decay_out,
                          cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    PL_REQUIRE(C > 0 && H > 0 && taps >= 1 && taps <= 64, "ssm_conv: bad sizes C=%d H=%d taps=%d", C, H, taps);
    const dim3 grid(num_seqs, (C + 31) / 32 + 1);
    if (dtype == PL_F32)
        ssm_conv_kernel<float><<<grid, 256, 0, stream>>>((const float*)zx, ld, c0, C, dt0, H, cw, cb, taps, dt_bias, a_log,
                                                         state, state_stride, cu_q, slots, xbc, dt_out, decay_out);
    else if (dtype == PL_BF16)
        ssm_conv_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)zx, ld, c0, C, dt0, H, cw, cb, taps,
                                                                 dt_bias, a_log, state, state_stride, cu_q, slots, xbc,
                                                                 dt_out, decay_out);
    else
        return pl_fail("ssm_conv: unknown dtype %d", dtype);
    PL_LAUNCHED("ssm_conv");
    return 0;
}

// ------------------------------------------------------------------ the recurrence
// grid: (requests, heads, blocks of 16 columns).  A column p of a head's state is independent of the others:
// eight lanes share it, each keeping NPER of its N values in registers (value n of lane l: n = l + 8 i), so a
// warp runs four columns and a block of 128 threads sixteen.  The tokens' B, C, x, dt and decay are staged
// in shared memory sixteen tokens at a time.
constexpr int SCAN_COLS = 16, SCAN_TOK = 16, SCAN_LANES = 8;

template <int NPER>
__global__ void __launch_bounds__(128) ssm_scan_kernel(const float* __restrict__ xbc, int C, int inner, int G, int N, int H,
                                                       int P, const float* __restrict__ dt, const float* __restrict__ decay,
                                                       const float* __restrict__ Dskip, float* __restrict__ state,
                                                       long long state_stride, long long ssm_off,
                                                       const int* __restrict__ cu_q, const int* __restrict__ slots,
                                                       float* __restrict__ y) {
    extern __shared__ float sm[];
    const int s = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * SCAN_COLS;
    const int slot = slots[s];
    const int q0 = cu_q[s], nq = cu_q[s + 1] - q0;
    if (slot < 0 || nq <= 0) return;
    float* Bs = sm;                                  // [SCAN_TOK][N]
    float* Cs = Bs + SCAN_TOK * N;                   // [SCAN_TOK][N]
    float* xs = Cs + SCAN_TOK * N;                   // [SCAN_TOK][SCAN_COLS]
    float* ds = xs + SCAN_TOK * SCAN_COLS;           // [SCAN_TOK][2]: dt, decay
    const int g = h / (H / G);
    const int lane = threadIdx.x & (SCAN_LANES - 1), col = threadIdx.x / SCAN_LANES;
    const int p = p0 + col;
    const bool ok = p < P;
    float* sp = state + (size_t)slot * state_stride + ssm_off + ((size_t)h * P + (ok ? p : 0)) * N;
    float S[NPER];
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        const int n = lane + SCAN_LANES * i;
        S[i] = ok && n < N ? sp[n] : 0.f;
    }
    const float dskip = __ldg(Dskip + h);
    const float* b_src = xbc + inner + (size_t)g * N;
    const float* c_src = xbc + inner + (size_t)G * N + (size_t)g * N;
    for (int t0 = 0; t0 < nq; t0 += SCAN_TOK) {
        const int nt = min(SCAN_TOK, nq - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * N; i += blockDim.x) {
            const int t = i / N, n = i - t * N;
            const size_t row = (size_t)(q0 + t0 + t) * C;
            Bs[i] = b_src[row + n];
            Cs[i] = c_src[row + n];
        }
        for (int i = threadIdx.x; i < nt * SCAN_COLS; i += blockDim.x) {
            const int t = i / SCAN_COLS, cc = i - t * SCAN_COLS;
            xs[i] = p0 + cc < P ? xbc[(size_t)(q0 + t0 + t) * C + (size_t)h * P + p0 + cc] : 0.f;
        }
        for (int i = threadIdx.x; i < nt; i += blockDim.x) {
            ds[2 * i] = dt[(size_t)(q0 + t0 + i) * H + h];
            ds[2 * i + 1] = decay[(size_t)(q0 + t0 + i) * H + h];
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float x = xs[t * SCAN_COLS + col];
            const float dtx = ds[2 * t] * x, a = ds[2 * t + 1];
            const float* Bt = Bs + t * N;
            const float* Ct = Cs + t * N;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < NPER; ++i) {
                const int n = lane + SCAN_LANES * i;
                if (n < N) {
                    S[i] = fmaf(a, S[i], dtx * Bt[n]);
                    acc = fmaf(S[i], Ct[n], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (lane == 0 && ok) y[(size_t)(q0 + t0 + t) * inner + (size_t)h * P + p] = fmaf(dskip, x, acc);
        }
    }
    if (ok) {
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
            const int n = lane + SCAN_LANES * i;
            if (n < N) sp[n] = S[i];
        }
    }
}

PL_EXPORT int pl_ssm_scan(const float* xbc, int C, int inner, int G, int N, int H, int P, const float* dt,
                          const float* decay, const float* Dskip, float* state, long long state_stride, long long ssm_off,
                          const int* cu_q, const int* slots, int num_seqs, float* y, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    PL_REQUIRE(G > 0 && H > 0 && H % G == 0 && N > 0 && P > 0 && inner == H * P && C == inner + 2 * G * N,
               "ssm_scan: bad sizes heads=%d groups=%d state=%d head size=%d", H, G, N, P);
    PL_REQUIRE(N <= 256, "ssm_scan: a state of %d values per column is more than the kernel keeps in registers (256)", N);
    const dim3 grid(num_seqs, H, (P + SCAN_COLS - 1) / SCAN_COLS);
    const size_t smem = ((size_t)2 * SCAN_TOK * N + SCAN_TOK * SCAN_COLS + 2 * SCAN_TOK) * sizeof(float);
    const int per = (N + SCAN_LANES - 1) / SCAN_LANES;
#define PL_SCAN(NP)                                                                                                       \
    ssm_scan_kernel<NP><<<grid, 128, smem, stream>>>(xbc, C, inner, G, N, H, P, dt, decay, Dskip, state, state_stride,   \
                                                     ssm_off, cu_q, slots, y)
    if (per <= 2) PL_SCAN(2);
    else if (per <= 4) PL_SCAN(4);
    else if (per <= 8) PL_SCAN(8);
    else if (per <= 16) PL_SCAN(16);
    else PL_SCAN(32);
#undef PL_SCAN
    PL_LAUNCHED("ssm_scan");
    return 0;
}

// ------------------------------------------------------------------ gate, then the norm in equal parts
// grid: (tokens, parts).  v = y * silu(z); out = v / sqrt(mean(v^2 over the part) + eps) * w.
template <typename T>
__global__ void __launch_bounds__(256) gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, int ldz,
                                                               const float* __restrict__ w, float eps, T* __restrict__ out,
                                                               int inner, int part, const int* __restrict__ token_seq) {
    __shared__ float red[32];
    const int t = blockIdx.x, c0 = blockIdx.y * part;
    if (token_seq != nullptr && token_seq[t] < 0) {              // a row that pads the step: nothing was computed for it
        for (int i = threadIdx.x; i < part; i += blockDim.x) out[(size_t)t * inner + c0 + i] = from_float<T>(0.f);
        return;
    }
    const float* yr = y + (size_t)t * inner + c0;
    const T* zr = z + (size_t)t * ldz + c0;
    float sq = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float v = yr[i] * silu_f(to_float(zr[i]));
        sq += v * v;
    }
    const float r = 1.0f / sqrtf(block_sum(sq, red) / (float)part + eps);
    T* o = out + (size_t)t * inner + c0;
    for (int i = threadIdx.x; i < part; i += blockDim.x)
        o[i] = from_float<T>(yr[i] * silu_f(to_float(zr[i])) * r * __ldg(w + c0 + i));
}

PL_EXPORT int pl_gated_group_norm(const float* y, const void* z, int dtype, int ldz, const float* w, float eps, void* out,
                                  int T, int inner, int groups, const int* token_seq, cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(groups > 0 && inner % groups == 0, "gated_group_norm: %d elements in %d parts", inner, groups);
    const dim3 grid(T, groups);
    if (dtype == PL_F32)
        gated_group_norm_kernel<float><<<grid, 256, 0, stream>>>(y, (const float*)z, ldz, w, eps, (float*)out, inner,
                                                                 inner / groups, token_seq);
    else if (dtype == PL_BF16)
        gated_group_norm_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(y, (const __nv_bfloat16*)z, ldz, w, eps,
                                                                         (__nv_bfloat16*)out, inner, inner / groups, token_seq);
    else
        return pl_fail("gated_group_norm: unknown dtype %d", dtype);
    PL_LAUNCHED("gated_group_norm");
    return 0;
}
