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
// grid: (requests, channel blocks + 1, token chunks).  A block of channels takes CONV_TOK tokens of its request
// (chunk z: tokens z * CONV_TOK ..; chunks behind the request's last token leave at once); the block of chunk 0
// is the only one that reads the request's old inputs, and it alone writes the new ones, after a barrier, from
// this step's inputs (which nobody writes) and the old ones it holds: no block waits for another.  The last
// block row of a request turns dt_in into dt and the decay.
// Threads: CL channel lanes x (256 / CL) token lanes; CL = 32 for prompt portions, 256 (one token lane) for
// steps of few tokens per request, where blocks of 32 channels would be mostly idle threads.
constexpr int CONV_TOK = 64;

template <typename T, int CL>
__global__ void __launch_bounds__(256) ssm_conv_kernel(const T* __restrict__ zx, int ld, int c0, int C, int dt0, int H,
                                                       const float* __restrict__ cw, const float* __restrict__ cb, int taps,
                                                       const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                                       float* __restrict__ state, long long state_stride,
                                                       const int* __restrict__ cu_q, const int* __restrict__ slots,
                                                       float* __restrict__ xbc, float* __restrict__ dt_out,
                                                       float* __restrict__ decay_out) {
    constexpr int TL = 256 / CL;
    const int s = blockIdx.x;
    const int slot = slots[s];
    const int q0 = cu_q[s], nq = cu_q[s + 1] - q0;
    const int t_lo = blockIdx.z * CONV_TOK, t_hi = min(nq, t_lo + CONV_TOK);
    if (slot < 0 || t_lo >= nq) return;
    const int cblocks = (C + CL - 1) / CL;
    if ((int)blockIdx.y == cblocks) {
        for (int i = threadIdx.x; i < (t_hi - t_lo) * H; i += blockDim.x) {
            const int t = t_lo + i / H, h = i % H;
            const float dt = softplus_f(to_float(zx[(size_t)(q0 + t) * ld + dt0 + h]) + __ldg(dt_bias + h));
            dt_out[(size_t)(q0 + t) * H + h] = dt;
            decay_out[(size_t)(q0 + t) * H + h] = expf(-expf(__ldg(a_log + h)) * dt);
        }
        return;
    }
    const int lane_c = threadIdx.x % CL, lane_t = threadIdx.x / CL;
    const int c = blockIdx.y * CL + lane_c;
    const bool ok = c < C;
    float* st = state + (size_t)slot * state_stride;              // [taps-1][C]
    const int hist = taps - 1;
    if (ok) {
        const float bias = __ldg(cb + c);
        const T* col = zx + (size_t)q0 * ld + c0 + c;
        auto input = [&](int src) { return src >= 0 ? to_float(col[(size_t)src * ld]) : st[(size_t)(hist + src) * C + c]; };
        if (taps <= 8 && CL == 32) {                 // (steps of a token or two per request: the plain loop below)
            // a token lane walks a run of consecutive tokens and keeps the last taps-1 inputs and the channel's
            // weights in registers: one load per output
            constexpr int PER = CONV_TOK / TL;
            const int ta = t_lo + lane_t * PER, tb = min(t_hi, ta + PER);
            float w[8], win[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                w[k] = k < taps ? __ldg(cw + (size_t)c * taps + k) : 0.f;      // w[k] multiplies the input k - hist back
                win[k] = 0.f;
            }
            if (ta < tb) {
#pragma unroll
                for (int k = 0; k < 7; ++k)
                    if (k < hist) win[k] = input(ta - hist + k);                // the inputs in front of the run
            }
            for (int t = ta; t < tb; ++t) {
                const float cur = to_float(col[(size_t)t * ld]);
                float acc = bias;
#pragma unroll
                for (int k = 0; k < 7; ++k)
                    if (k < hist) acc = fmaf(w[k], win[k], acc);
                // the current token's weight is the last column
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (k == hist) acc = fmaf(w[k], cur, acc);
                xbc[(size_t)(q0 + t) * C + c] = silu_f(acc);
#pragma unroll
                for (int k = 0; k < 7; ++k)
                    if (k + 1 < hist) win[k] = win[k + 1];
#pragma unroll
                for (int k = 0; k < 7; ++k)
                    if (k == hist - 1) win[k] = cur;
            }
        } else {
            for (int t = t_lo + lane_t; t < t_hi; t += TL) {
                float acc = bias;
                for (int k = 0; k < taps; ++k) acc = fmaf(__ldg(cw + (size_t)c * taps + k), input(t - hist + k), acc);
                xbc[(size_t)(q0 + t) * C + c] = silu_f(acc);
            }
        }
    }
    if (blockIdx.z != 0) return;
    __syncthreads();                                                // every read of the old inputs is done
    if (ok && lane_t == 0) {
        // the last taps-1 inputs of [old inputs ; this step's inputs]: a pass in place from the front is safe,
        // since entry j reads old entry j + nq > j or a new input
        const T* col = zx + (size_t)q0 * ld + c0 + c;
        for (int j = 0; j < hist; ++j) {
            const int src = nq + j - hist;                          // index among this step's inputs
            st[(size_t)j * C + c] = src >= 0 ? to_float(col[(size_t)src * ld]) : st[(size_t)(j + nq) * C + c];
        }
    }
}

// `max_tokens`: no request of the step brings more (the step's token count will do).
PL_EXPORT int pl_ssm_conv(const void* zx, int dtype, int ld, int c0, int C, int dt0, int H, const float* cw, const float* cb,
                          int taps, const float* dt_bias, const float* a_log, float* state, long long state_stride,
                          const int* cu_q, const int* slots, int num_seqs, int max_tokens, float* xbc, float* dt_out,
                          float* decay_out, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    PL_REQUIRE(C > 0 && H > 0 && taps >= 1 && taps <= 64 && max_tokens >= 1, "ssm_conv: bad sizes C=%d H=%d taps=%d", C, H, taps);
    const bool few = max_tokens <= 2 * num_seqs;                   // a decode step, or nearly
    const int CL = few ? 256 : 32;
    const dim3 grid(num_seqs, (C + CL - 1) / CL + 1, (max_tokens + CONV_TOK - 1) / CONV_TOK);
    PL_REQUIRE(grid.z <= 65535, "ssm_conv: %d tokens in a step", max_tokens);
#define PL_CONV(TT, L)                                                                                                    \
    ssm_conv_kernel<TT, L><<<grid, 256, 0, stream>>>((const TT*)zx, ld, c0, C, dt0, H, cw, cb, taps, dt_bias, a_log, state, \
                                                     state_stride, cu_q, slots, xbc, dt_out, decay_out)
    if (dtype == PL_F32) {
        if (few) PL_CONV(float, 256); else PL_CONV(float, 32);
    } else if (dtype == PL_BF16) {
        if (few) PL_CONV(__nv_bfloat16, 256); else PL_CONV(__nv_bfloat16, 32);
    } else {
        return pl_fail("ssm_conv: unknown dtype %d", dtype);
    }
#undef PL_CONV
    PL_LAUNCHED("ssm_conv");
    return 0;
}

// ------------------------------------------------------------------ the recurrence
// grid: (requests, heads, blocks of columns).  A column p of a head's state is independent of the others:
// eight or sixteen lanes share it, each keeping NPER of its N values in registers, and a block of 128 threads
// runs sixteen or eight columns.  The tokens' B, C, x, dt and decay come into shared memory sixteen tokens at a time by
// asynchronous copies, two chunks in flight: the copies of the next chunk run while this one is computed.  Per
// token a lane does 2 NPER multiply-adds and keeps its part of the token's output; the parts of the sixteen
// tokens are summed over the lanes together at the end of the chunk, so the only chain from token to token
// is the state's own multiply-add.
// VEC (N, the row of xBC and the head size are multiples of four): 16-byte copies and reads; lane l holds the
// values n = (lanes j + l) * 4 + k, so that the lanes' reads of shared memory and of the state are contiguous.
// Otherwise 4-byte copies and n = l + 8 i.
constexpr int SCAN_TOK = 16;

__device__ __forceinline__ void cp_async_f(float* dst, const float* src, bool ok) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
                 "r"(ok ? 4 : 0));
}
__device__ __forceinline__ void cp_async_f4(float* dst, const float* src, bool ok) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
                 "r"(ok ? 16 : 0));
}

template <int NPER, bool VEC, int SCAN_LANES>
__global__ void __launch_bounds__(128) ssm_scan_kernel(const float* __restrict__ xbc, int C, int inner, int G, int N, int H,
                                                       int P, const float* __restrict__ dt, const float* __restrict__ decay,
                                                       const float* __restrict__ Dskip, float* __restrict__ state,
                                                       long long state_stride, long long ssm_off,
                                                       const int* __restrict__ cu_q, const int* __restrict__ slots,
                                                       float* __restrict__ y) {
    extern __shared__ __align__(16) float sm[];
    constexpr int SCAN_COLS = 128 / SCAN_LANES;                     // columns of a block
    constexpr int ROW = SCAN_LANES * NPER;                          // a token's B (or C), zeros from N on
    constexpr int STAGE = 2 * SCAN_TOK * ROW + SCAN_TOK * SCAN_COLS + 2 * SCAN_TOK;
    const int s = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * SCAN_COLS;
    const int slot = slots[s];
    const int q0 = cu_q[s], nq = cu_q[s + 1] - q0;
    if (slot < 0 || nq <= 0) return;
    const int g = h / (H / G);
    const int tid = threadIdx.x, lane = tid & (SCAN_LANES - 1), col = tid / SCAN_LANES;
    const int p = p0 + col;
    const bool ok = p < P;
    const float* b_src = xbc + inner + (size_t)g * N;
    const float* c_src = xbc + inner + (size_t)G * N + (size_t)g * N;
    const float* x_src = xbc + (size_t)h * P + p0;

    // every position of a stage is written by a copy (zero-filled where there is nothing to copy)
    auto issue = [&](int stage, int t0) {
        float* Bs = sm + stage * STAGE;
        float* Cs = Bs + SCAN_TOK * ROW;
        float* xs = Cs + SCAN_TOK * ROW;
        float* ds = xs + SCAN_TOK * SCAN_COLS;
        const int nt = min(SCAN_TOK, nq - t0);
        if (VEC) {
#pragma unroll
            for (int i = tid; i < SCAN_TOK * ROW / 4; i += 128) {
                const int t = i / (ROW / 4), n = (i - t * (ROW / 4)) * 4;
                const bool in = t < nt && n < N;
                const size_t row = (size_t)(q0 + t0 + (t < nt ? t : 0)) * C + (in ? n : 0);
                cp_async_f4(Bs + t * ROW + n, b_src + row, in);
                cp_async_f4(Cs + t * ROW + n, c_src + row, in);
            }
        } else {
#pragma unroll
            for (int i = tid; i < SCAN_TOK * ROW; i += 128) {
                const int t = i / ROW, n = i - t * ROW;
                const bool in = t < nt && n < N;
                const size_t row = (size_t)(q0 + t0 + (t < nt ? t : 0)) * C + (in ? n : 0);
                cp_async_f(Bs + t * ROW + n, b_src + row, in);
                cp_async_f(Cs + t * ROW + n, c_src + row, in);
            }
        }
#pragma unroll
        for (int i = tid; i < SCAN_TOK * SCAN_COLS; i += 128) {
            const int t = i / SCAN_COLS, cc = i - t * SCAN_COLS;
            const bool in = t < nt && p0 + cc < P;
            cp_async_f(xs + i, x_src + (size_t)(q0 + t0 + (t < nt ? t : 0)) * C + (in ? cc : 0), in);
        }
        if (tid < 2 * SCAN_TOK) {
            const int t = tid >> 1;
            const bool in = t < nt;
            cp_async_f(ds + tid, ((tid & 1) ? decay : dt) + (size_t)(q0 + t0 + (in ? t : 0)) * H + h, in);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    issue(0, 0);
    float* sp = state + (size_t)slot * state_stride + ssm_off + ((size_t)h * P + (ok ? p : 0)) * N;
    float S[NPER];
    if (VEC) {
#pragma unroll
        for (int j = 0; j < NPER / 4; ++j) {
            const int n = (j * SCAN_LANES + lane) * 4;
            const float4 v = ok && n < N ? *reinterpret_cast<const float4*>(sp + n) : make_float4(0.f, 0.f, 0.f, 0.f);
            S[4 * j] = v.x, S[4 * j + 1] = v.y, S[4 * j + 2] = v.z, S[4 * j + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < NPER; ++i) S[i] = ok && lane + SCAN_LANES * i < N ? sp[lane + SCAN_LANES * i] : 0.f;
    }
    const float dskip = __ldg(Dskip + h);
    const int n_chunks = (nq + SCAN_TOK - 1) / SCAN_TOK;
    for (int k = 0; k < n_chunks; ++k) {
        const int t0 = k * SCAN_TOK;
        const int nt = min(SCAN_TOK, nq - t0);
        if (k + 1 < n_chunks) {
            issue((k + 1) & 1, t0 + SCAN_TOK);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        const float* Bs = sm + (k & 1) * STAGE;
        const float* Cs = Bs + SCAN_TOK * ROW;
        const float* xs = Cs + SCAN_TOK * ROW;
        const float* ds = xs + SCAN_TOK * SCAN_COLS;
        float part[SCAN_TOK];
#pragma unroll
        for (int t = 0; t < SCAN_TOK; ++t) {
            // (a token behind the request's last has dt = 0 and decay = 0 in shared memory; it is skipped so
            // that the state stays what the last real token left)
            part[t] = 0.f;
            if (t < nt) {
                const float dtx = ds[2 * t] * xs[t * SCAN_COLS + col], a = ds[2 * t + 1];
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                if (VEC) {
#pragma unroll
                    for (int j = 0; j < NPER / 4; ++j) {
                        const int n = (j * SCAN_LANES + lane) * 4;
                        const float4 b = *reinterpret_cast<const float4*>(Bs + t * ROW + n);
                        const float4 c = *reinterpret_cast<const float4*>(Cs + t * ROW + n);
                        S[4 * j] = fmaf(a, S[4 * j], dtx * b.x);
                        S[4 * j + 1] = fmaf(a, S[4 * j + 1], dtx * b.y);
                        S[4 * j + 2] = fmaf(a, S[4 * j + 2], dtx * b.z);
                        S[4 * j + 3] = fmaf(a, S[4 * j + 3], dtx * b.w);
                        acc[0] = fmaf(S[4 * j], c.x, acc[0]);
                        acc[1] = fmaf(S[4 * j + 1], c.y, acc[1]);
                        acc[2] = fmaf(S[4 * j + 2], c.z, acc[2]);
                        acc[3] = fmaf(S[4 * j + 3], c.w, acc[3]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < NPER; ++i) {
                        const int n = lane + SCAN_LANES * i;
                        S[i] = fmaf(a, S[i], dtx * Bs[t * ROW + n]);
                        acc[i & 3] = fmaf(S[i], Cs[t * ROW + n], acc[i & 3]);
                    }
                }
                part[t] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            }
        }
        // the lanes' parts of sixteen tokens: at every exchange a lane hands half of the tokens it is still
        // responsible for to its partner and takes the partner's parts of the other half, so that after
        // log2(lanes) exchanges it holds the full sums of 16 / lanes tokens, the first of which is token `tb`
        int tb = 0;
        {
            int cnt = SCAN_TOK;
#pragma unroll
            for (int m = SCAN_LANES / 2; m >= 1; m >>= 1) {
                cnt >>= 1;
                const bool upper = lane & m;
#pragma unroll
                for (int t = 0; t < SCAN_TOK / 2; ++t) {
                    if (t < cnt) {
                        const float give = upper ? part[t] : part[t + cnt], keep = upper ? part[t + cnt] : part[t];
                        part[t] = keep + __shfl_xor_sync(0xffffffffu, give, m);
                    }
                }
                tb += upper ? cnt : 0;
            }
        }
#pragma unroll
        for (int e = 0; e < SCAN_TOK / SCAN_LANES; ++e) {
            const int t = tb + e;
            if (ok && t < nt)
                y[(size_t)(q0 + t0 + t) * inner + (size_t)h * P + p] = fmaf(dskip, xs[t * SCAN_COLS + col], part[e]);
        }
        __syncthreads();                                           // the stage is free for the chunk after next
    }
    if (ok) {
        if (VEC) {
#pragma unroll
            for (int j = 0; j < NPER / 4; ++j) {
                const int n = (j * SCAN_LANES + lane) * 4;
                if (n < N) *reinterpret_cast<float4*>(sp + n) = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < NPER; ++i)
                if (lane + SCAN_LANES * i < N) sp[lane + SCAN_LANES * i] = S[i];
        }
    }
}

// The same recurrence with the state values of FOUR columns per thread (N, the row of xBC and the state's
// layout allow 16-byte accesses).  In the kernel above every column's lanes read all of B_t and C_t from shared
// memory for two multiply-adds per value read, and shared memory, not the multiply-adds, sets the pace; here a
// group of LPG lanes owns four columns, a lane keeps the values n = (LPG v + lane) * 4 + k (v < NV, k < 4) of all
// four, and a 16-byte read of B_t and of C_t feeds 32 multiply-adds.  A block of 128 threads runs 512 / LPG
// columns.  The 64 partial outputs of a chunk (16 tokens x 4 columns) are summed over the group's lanes together.
template <int LPG, int NV>
__global__ void __launch_bounds__(128) ssm_scan4_kernel(const float* __restrict__ xbc, int C, int inner, int G, int N, int H,
                                                        int P, const float* __restrict__ dt, const float* __restrict__ decay,
                                                        const float* __restrict__ Dskip, float* __restrict__ state,
                                                        long long state_stride, long long ssm_off,
                                                        const int* __restrict__ cu_q, const int* __restrict__ slots,
                                                        float* __restrict__ y) {
    extern __shared__ __align__(16) float sm[];
    constexpr int COLS = 512 / LPG;                                 // columns of a block
    constexpr int ROW = LPG * NV * 4;                               // a token's B (or C), zeros from N on
    constexpr int STAGE = 2 * SCAN_TOK * ROW + SCAN_TOK * COLS + 2 * SCAN_TOK;
    const int s = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * COLS;
    const int slot = slots[s];
    const int q0 = cu_q[s], nq = cu_q[s + 1] - q0;
    if (slot < 0 || nq <= 0) return;
    const int g = h / (H / G);
    const int tid = threadIdx.x, lane = tid & (LPG - 1), grp = tid / LPG;
    const int pc = p0 + grp * 4;                                    // the group's first column
    const float* b_src = xbc + inner + (size_t)g * N;
    const float* c_src = xbc + inner + (size_t)G * N + (size_t)g * N;
    const float* x_src = xbc + (size_t)h * P + p0;

    auto issue = [&](int stage, int t0) {
        float* Bs = sm + stage * STAGE;
        float* Cs = Bs + SCAN_TOK * ROW;
        float* xs = Cs + SCAN_TOK * ROW;
        float* ds = xs + SCAN_TOK * COLS;
        const int nt = min(SCAN_TOK, nq - t0);
        // (tokens behind the chunk's last are never read: nothing is copied for them)
#pragma unroll
        for (int i = tid; i < SCAN_TOK * ROW / 4; i += 128) {
            const int t = i / (ROW / 4), n = (i - t * (ROW / 4)) * 4;
            if (t >= nt) break;
            const bool in = n < N;
            const size_t row = (size_t)(q0 + t0 + t) * C + (in ? n : 0);
            cp_async_f4(Bs + t * ROW + n, b_src + row, in);
            cp_async_f4(Cs + t * ROW + n, c_src + row, in);
        }
#pragma unroll
        for (int i = tid; i < SCAN_TOK * COLS; i += 128) {
            const int t = i / COLS, cc = i - t * COLS;
            if (t >= nt) break;
            const bool in = p0 + cc < P;
            cp_async_f(xs + i, x_src + (size_t)(q0 + t0 + t) * C + (in ? cc : 0), in);
        }
        if (tid < 2 * SCAN_TOK) {
            const int t = tid >> 1;
            const bool in = t < nt;
            cp_async_f(ds + tid, ((tid & 1) ? decay : dt) + (size_t)(q0 + t0 + (in ? t : 0)) * H + h, in);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    issue(0, 0);
    float* sp = state + (size_t)slot * state_stride + ssm_off + (size_t)h * P * N;
    float S[4][NV * 4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int n = (v * LPG + lane) * 4;
            const float4 val = pc + c < P && n < N ? *reinterpret_cast<const float4*>(sp + (size_t)(pc + c) * N + n)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
            S[c][4 * v] = val.x, S[c][4 * v + 1] = val.y, S[c][4 * v + 2] = val.z, S[c][4 * v + 3] = val.w;
        }
    const float dskip = __ldg(Dskip + h);
    const int n_chunks = (nq + SCAN_TOK - 1) / SCAN_TOK;
    for (int k = 0; k < n_chunks; ++k) {
        const int t0 = k * SCAN_TOK;
        const int nt = min(SCAN_TOK, nq - t0);
        if (k + 1 < n_chunks) {
            issue((k + 1) & 1, t0 + SCAN_TOK);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        const float* Bs = sm + (k & 1) * STAGE;
        const float* Cs = Bs + SCAN_TOK * ROW;
        const float* xs = Cs + SCAN_TOK * ROW;
        const float* ds = xs + SCAN_TOK * COLS;
        float part[SCAN_TOK * 4];                                   // [token][column]
#pragma unroll
        for (int t = 0; t < SCAN_TOK; ++t) {
#pragma unroll
            for (int c = 0; c < 4; ++c) part[4 * t + c] = 0.f;
            if (t < nt) {                                           // (the state stays what the last real token left)
                const float4 x4 = *reinterpret_cast<const float4*>(xs + t * COLS + grp * 4);
                const float dtv = ds[2 * t], a = ds[2 * t + 1];
                const float dtx[4] = {dtv * x4.x, dtv * x4.y, dtv * x4.z, dtv * x4.w};
#pragma unroll
                for (int v = 0; v < NV; ++v) {
                    const int n = (v * LPG + lane) * 4;
                    const float4 b = *reinterpret_cast<const float4*>(Bs + t * ROW + n);
                    const float4 cc = *reinterpret_cast<const float4*>(Cs + t * ROW + n);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float* Sc = S[c] + 4 * v;
                        Sc[0] = fmaf(a, Sc[0], dtx[c] * b.x);
                        Sc[1] = fmaf(a, Sc[1], dtx[c] * b.y);
                        Sc[2] = fmaf(a, Sc[2], dtx[c] * b.z);
                        Sc[3] = fmaf(a, Sc[3], dtx[c] * b.w);
                        part[4 * t + c] = fmaf(Sc[3], cc.w, fmaf(Sc[2], cc.z, fmaf(Sc[1], cc.y, fmaf(Sc[0], cc.x, part[4 * t + c]))));
                    }
                }
            }
        }
        // the group's lanes' parts of 64 outputs: at every exchange a lane hands half of the outputs it is still
        // responsible for to its partner and takes the partner's parts of the other half
        int first = 0;
        if (nt == 1) {
            // one token (a decode step): the four outputs by a plain exchange over the group, every lane gets all
#pragma unroll
            for (int m = LPG / 2; m >= 1; m >>= 1)
#pragma unroll
                for (int c = 0; c < 4; ++c) part[c] += __shfl_xor_sync(0xffffffffu, part[c], m);
            if (lane < 4 && pc + lane < P) {
                const float v = lane == 0 ? part[0] : lane == 1 ? part[1] : lane == 2 ? part[2] : part[3];
                y[(size_t)(q0 + t0) * inner + (size_t)h * P + pc + lane] = fmaf(dskip, xs[grp * 4 + lane], v);
            }
        } else {
            int cnt = SCAN_TOK * 4;
#pragma unroll
            for (int m = LPG / 2; m >= 1; m >>= 1) {
                cnt >>= 1;
                const bool upper = lane & m;
#pragma unroll
                for (int i = 0; i < SCAN_TOK * 2; ++i) {
                    if (i < cnt) {
                        const float give = upper ? part[i] : part[i + cnt], keep = upper ? part[i + cnt] : part[i];
                        part[i] = keep + __shfl_xor_sync(0xffffffffu, give, m);
                    }
                }
                first += upper ? cnt : 0;
            }
#pragma unroll
            for (int e = 0; e < SCAN_TOK * 4 / LPG; ++e) {
                const int o = first + e, t = o >> 2, c = o & 3;
                if (pc + c < P && t < nt)
                    y[(size_t)(q0 + t0 + t) * inner + (size_t)h * P + pc + c] = fmaf(dskip, xs[t * COLS + grp * 4 + c], part[e]);
            }
        }
        __syncthreads();                                           // the stage is free for the chunk after next
    }
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int n = (v * LPG + lane) * 4;
            if (pc + c < P && n < N)
                *reinterpret_cast<float4*>(sp + (size_t)(pc + c) * N + n) =
                    make_float4(S[c][4 * v], S[c][4 * v + 1], S[c][4 * v + 2], S[c][4 * v + 3]);
        }
}

template <int LPG, int NV>
static int launch_scan4(const float* xbc, int C, int inner, int G, int N, int H, int P, const float* dt, const float* decay,
                        const float* Dskip, float* state, long long state_stride, long long ssm_off, const int* cu_q,
                        const int* slots, int num_seqs, float* y, cudaStream_t stream) {
    constexpr int COLS = 512 / LPG;
    const size_t smem = (size_t)2 * (2 * SCAN_TOK * LPG * NV * 4 + SCAN_TOK * COLS + 2 * SCAN_TOK) * sizeof(float);
    auto kernel = ssm_scan4_kernel<LPG, NV>;
    static bool attr_set = false;
    if (smem > 48 * 1024 && !attr_set) {
        PL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    kernel<<<dim3(num_seqs, H, (P + COLS - 1) / COLS), 128, smem, stream>>>(xbc, C, inner, G, N, H, P, dt, decay, Dskip, state,
                                                                           state_stride, ssm_off, cu_q, slots, y);
    PL_LAUNCHED("ssm_scan");
    return 0;
}

// `max_tokens`: no request of the step brings more (the step's token count will do).
PL_EXPORT int pl_ssm_scan(const float* xbc, int C, int inner, int G, int N, int H, int P, const float* dt,
                          const float* decay, const float* Dskip, float* state, long long state_stride, long long ssm_off,
                          const int* cu_q, const int* slots, int num_seqs, int max_tokens, float* y, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    PL_REQUIRE(G > 0 && H > 0 && H % G == 0 && N > 0 && P > 0 && inner == H * P && C == inner + 2 * G * N,
               "ssm_scan: bad sizes heads=%d groups=%d state=%d head size=%d", H, G, N, P);
    PL_REQUIRE(N <= 256, "ssm_scan: a state of %d values per column is more than the kernel keeps in registers (256)", N);
    const bool vec4 = N % 4 == 0 && C % 4 == 0 && inner % 4 == 0 && P % 4 == 0 && state_stride % 4 == 0 && ssm_off % 4 == 0 &&
                      (((uintptr_t)xbc | (uintptr_t)state) & 15) == 0;
    // Prompt portions: four columns per thread.  Steps of a token or two per request are bound by reading and
    // writing the state, and the kernel with a column per eight lanes, which needs half the registers, keeps more
    // of those accesses in flight (64 requests at 64 heads x 64 x 128: 56 against 85 us).
    const bool few = max_tokens <= 2 * num_seqs;
    if (vec4 && !few) {
#define PL_SCAN4(L, V) return launch_scan4<L, V>(xbc, C, inner, G, N, H, P, dt, decay, Dskip, state, state_stride, ssm_off, cu_q, slots, num_seqs, y, stream)
        if (N <= 16) PL_SCAN4(4, 1);
        if (N <= 32) PL_SCAN4(8, 1);
        if (N <= 64) PL_SCAN4(16, 1);
        if (N <= 128) PL_SCAN4(32, 1);
        PL_SCAN4(32, 2);
#undef PL_SCAN4
    }
    // (sixteen lanes per column were tried for 64 state values and more: slower in prompts and in decoding)
    const int lanes = 8;
    const dim3 grid(num_seqs, H, (P + 128 / lanes - 1) / (128 / lanes));
    const int per = (N + lanes - 1) / lanes;
    const bool vec = N % 4 == 0 && C % 4 == 0 && inner % 4 == 0 && state_stride % 4 == 0 && ssm_off % 4 == 0 &&
                     (((uintptr_t)xbc | (uintptr_t)state) & 15) == 0;
#define PL_SCAN(NP, V, L)                                                                                                  \
    do {                                                                                                                   \
        const size_t smem = (size_t)2 * (2 * SCAN_TOK * L * NP + SCAN_TOK * (128 / L) + 2 * SCAN_TOK) * sizeof(float);     \
        auto kernel = ssm_scan_kernel<NP, V, L>;                                                                           \
        static bool attr_set = false;                                                                                      \
        if (smem > 48 * 1024 && !attr_set) {                                                                               \
            PL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                 \
            attr_set = true;                                                                                               \
        }                                                                                                                  \
        kernel<<<grid, 128, smem, stream>>>(xbc, C, inner, G, N, H, P, dt, decay, Dskip, state, state_stride, ssm_off, cu_q, \
                                            slots, y);                                                                     \
    } while (0)
    if (vec && per > 2) {
        if (per <= 4) PL_SCAN(4, true, 8);
        else if (per <= 8) PL_SCAN(8, true, 8);
        else if (per <= 16) PL_SCAN(16, true, 8);
        else PL_SCAN(32, true, 8);
    } else {
        if (per <= 2) PL_SCAN(2, false, 8);
        else if (per <= 4) PL_SCAN(4, false, 8);
        else if (per <= 8) PL_SCAN(8, false, 8);
        else if (per <= 16) PL_SCAN(16, false, 8);
        else PL_SCAN(32, false, 8);
    }
#undef PL_SCAN
    PL_LAUNCHED("ssm_scan");
    return 0;
}

// ------------------------------------------------------------------ gate, then the norm in equal parts
// grid: (tokens, parts).  v = y * silu(z); out = v / sqrt(mean(v^2 over the part) + eps) * w.
template <typename T> struct Quad;
template <> struct Quad<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Quad<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

// VEC: four elements per step (the part, the row strides and the pointers allow 16-byte accesses).
template <typename T, bool VEC>
__global__ void __launch_bounds__(512) gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, int ldz,
                                                               const float* __restrict__ w, float eps, T* __restrict__ out,
                                                               int inner, int part, const int* __restrict__ token_seq) {
    __shared__ float red[32];
    const int t = blockIdx.x, c0 = blockIdx.y * part;
    T* o = out + (size_t)t * inner + c0;
    if (token_seq != nullptr && token_seq[t] < 0) {              // a row that pads the step: nothing was computed for it
        for (int i = threadIdx.x; i < part; i += blockDim.x) o[i] = from_float<T>(0.f);
        return;
    }
    const float* yr = y + (size_t)t * inner + c0;
    const T* zr = z + (size_t)t * ldz + c0;
    float sq = 0.f;
    if (VEC && part <= (int)blockDim.x * 16) {
        // the gated row stays in registers between the sum of squares and the scaling: y and z are read once
        float4 keep[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * 4;
            keep[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < part) {
                const float4 a = Quad<float>::load(yr + i), g = Quad<T>::load(zr + i);
                keep[j] = make_float4(a.x * silu_f(g.x), a.y * silu_f(g.y), a.z * silu_f(g.z), a.w * silu_f(g.w));
                sq += (keep[j].x * keep[j].x + keep[j].y * keep[j].y) + (keep[j].z * keep[j].z + keep[j].w * keep[j].w);
            }
        }
        const float r = 1.0f / sqrtf(block_sum(sq, red) / (float)part + eps);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * 4;
            if (i < part) {
                const float4 ww = Quad<float>::load(w + c0 + i);
                Quad<T>::store(o + i, make_float4(keep[j].x * r * ww.x, keep[j].y * r * ww.y, keep[j].z * r * ww.z, keep[j].w * r * ww.w));
            }
        }
        return;
    }
    if (VEC) {
        for (int i = threadIdx.x * 4; i < part; i += blockDim.x * 4) {
            const float4 a = Quad<float>::load(yr + i), g = Quad<T>::load(zr + i);
            const float v0 = a.x * silu_f(g.x), v1 = a.y * silu_f(g.y), v2 = a.z * silu_f(g.z), v3 = a.w * silu_f(g.w);
            sq += (v0 * v0 + v1 * v1) + (v2 * v2 + v3 * v3);
        }
    } else {
        for (int i = threadIdx.x; i < part; i += blockDim.x) {
            const float v = yr[i] * silu_f(to_float(zr[i]));
            sq += v * v;
        }
    }
    const float r = 1.0f / sqrtf(block_sum(sq, red) / (float)part + eps);
    if (VEC) {
        for (int i = threadIdx.x * 4; i < part; i += blockDim.x * 4) {
            const float4 a = Quad<float>::load(yr + i), g = Quad<T>::load(zr + i), ww = Quad<float>::load(w + c0 + i);
            Quad<T>::store(o + i, make_float4(a.x * silu_f(g.x) * r * ww.x, a.y * silu_f(g.y) * r * ww.y,
                                              a.z * silu_f(g.z) * r * ww.z, a.w * silu_f(g.w) * r * ww.w));
        }
    } else {
        for (int i = threadIdx.x; i < part; i += blockDim.x)
            o[i] = from_float<T>(yr[i] * silu_f(to_float(zr[i])) * r * __ldg(w + c0 + i));
    }
}

PL_EXPORT int pl_gated_group_norm(const float* y, const void* z, int dtype, int ldz, const float* w, float eps, void* out,
                                  int T, int inner, int groups, const int* token_seq, cudaStream_t stream) {
    if (T == 0) return 0;
    PL_REQUIRE(groups > 0 && inner % groups == 0, "gated_group_norm: %d elements in %d parts", inner, groups);
    const dim3 grid(T, groups);
    const int part = inner / groups;
    const bool vec = part % 4 == 0 && ldz % 4 == 0 && inner % 4 == 0 && (((uintptr_t)y | (uintptr_t)z | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    const int threads = part >= 2048 ? 512 : (part >= 512 ? 256 : 128);
#define PL_GGN(TT, V)                                                                                                  \
    gated_group_norm_kernel<TT, V><<<grid, threads, 0, stream>>>(y, (const TT*)z, ldz, w, eps, (TT*)out, inner, part, token_seq)
    if (dtype == PL_F32) {
        if (vec) PL_GGN(float, true); else PL_GGN(float, false);
    } else if (dtype == PL_BF16) {
        if (vec) PL_GGN(__nv_bfloat16, true); else PL_GGN(__nv_bfloat16, false);
    } else {
        return pl_fail("gated_group_norm: unknown dtype %d", dtype);
    }
#undef PL_GGN
    PL_LAUNCHED("gated_group_norm");
    return 0;
}
