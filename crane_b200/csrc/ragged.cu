// Ragged-batch kernels (see ragged.cuh).  Everything here is f32 arithmetic on CUDA cores: norms, softmax, routers, the
// recurrent state and all that enters the recurrence are kept in 32-bit; the big linears run on the tensor cores (gemm.cu) from
// the bf16 planes these kernels emit, or through linear_f32_kernel in the exact mode.
//
// A row's result depends on that row's sequence only: every reduction runs in an order fixed by the row's own position and the
// launch constants, never by what else shares the step.
#include "ragged.cuh"
#include "decode.cuh"

namespace cb {

namespace {

__device__ __forceinline__ void store_act(const ActOut& o, int r, int c, float v) {
    if (o.f) o.f[(size_t)r * o.ldf + c] = v;
    if (o.hi) {
        const bf16 h = __float2bfloat16_rn(v);
        bf16* p = o.hi + (size_t)r * o.ldb + c;
        *p = h;
        if (o.lo_off) p[o.lo_off] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
}

template <typename KT> __device__ __forceinline__ float kv_load(const KT* p);
template <> __device__ __forceinline__ float kv_load<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float kv_load<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename KT> __device__ __forceinline__ void kv_store(KT* p, float v);
template <> __device__ __forceinline__ void kv_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void kv_store<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// ---------------------------------------------------------------------------------------------------------------- rows
__global__ void embed_scale_rows_kernel(const int* __restrict__ ids, int T, const bf16* __restrict__ embed, int W, float scale,
                                        float* __restrict__ x, int ldx) {
    const int r = blockIdx.x;
    const bf16* e = embed + (size_t)ids[r] * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) x[(size_t)r * ldx + c] = __bfloat162float(e[c]) * scale;
}

__global__ void dyt_rows_kernel(const float* __restrict__ x, int ldx, const int* __restrict__ rows, int W, const float* __restrict__ alpha,
                                const float* __restrict__ w, const float* __restrict__ b, ActOut out) {
    const int r = blockIdx.x, src = rows ? rows[r] : r;
    const float a = *alpha;
    for (int c = threadIdx.x; c < W; c += blockDim.x) store_act(out, r, c, tanhf(a * x[(size_t)src * ldx + c]) * w[c] + b[c]);
}

__global__ void gather_rows_kernel(const float* __restrict__ src, int lds, const int* __restrict__ rows, int W, float* __restrict__ dst, int ldd) {
    const int r = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) dst[(size_t)r * ldd + c] = src[(size_t)rows[r] * lds + c];
}

// ---------------------------------------------------------------------------------------------------------------- exact linear
// 64 x 64 output tile, 16-wide k-steps, 256 threads x (4 x 4) accumulators; each output element sums k = 0 .. K-1 in order.
template <int MODE>
__global__ void __launch_bounds__(256) linear_f32_kernel(const float* __restrict__ A, int lda, const bf16* __restrict__ Wt, int ldw, int M, int N,
                                                         int K, float* __restrict__ C, int ldc) {
    __shared__ float sa[16][64 + 4], sw[16][64 + 4];
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64, tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = tid; i < 64 * 16; i += 256) {
            const int r = i >> 4, k = i & 15;
            sa[k][r] = (m0 + r < M && k0 + k < K) ? A[(size_t)(m0 + r) * lda + k0 + k] : 0.f;
            sw[k][r] = (n0 + r < N && k0 + k < K) ? __bfloat162float(Wt[(size_t)(n0 + r) * ldw + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = sa[k][ty * 4 + i]; wv[i] = sw[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) {
                float* p = C + (size_t)m * ldc + n;
                *p = (MODE == LIN_RESID) ? *p + acc[i][j] : acc[i][j];
            }
        }
}

// ---------------------------------------------------------------------------------------------------------------- attention
// One warp per (row, head): q -> q / rms(q) * temp(pos); k -> k / rms(k) into its page; v into its page.
template <typename KT>
__global__ void attn_prep_kernel(RaggedBatch rb, AttnPrepArgs a) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int e = rb.row_entry[r], pos = rb.row_pos[r], slot = rb.ent_slot[e];
    const float* row = a.qkv + (size_t)r * a.ld;
    const int nheads = a.H + (a.has_kv ? 2 * a.G : 0);
    float temp = 1.f;
    if (a.temp_every > 0) temp = 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every) + 1.f);
    const int page = a.has_kv ? a.block_table[(size_t)slot * a.max_pages + pos / KV_PAGE] : 0;
    for (int hh = warp; hh < nheads; hh += nw) {
        if (hh < a.H + a.G) {            // q or k head: unit RMS over d
            const bool isq = hh < a.H;
            const float* src = row + (size_t)hh * a.d;
            float ss = 0.f;
            for (int c = lane; c < a.d; c += 32) ss += src[c] * src[c];
            ss = warp_sum(ss);
            const float inv = 1.f / sqrtf(ss / (float)a.d + a.eps) * (isq ? temp : 1.f);
            if (isq) {
                float* dst = a.q_out + (size_t)r * a.ldq + (size_t)hh * a.d;
                for (int c = lane; c < a.d; c += 32) dst[c] = src[c] * inv;
            } else {
                const int g = hh - a.H;
                KT* dst = (KT*)a.k_pool + (((size_t)page * a.G + g) * KV_PAGE + (pos % KV_PAGE)) * a.d;
                for (int c = lane; c < a.d; c += 32) kv_store<KT>(dst + c, src[c] * inv);
            }
        } else {
            const int g = hh - a.H - a.G;
            const float* src = row + (size_t)(a.H + a.G) * a.d + (size_t)g * a.dv;
            KT* dst = (KT*)a.v_pool + (((size_t)page * a.G + g) * KV_PAGE + (pos % KV_PAGE)) * a.dv;
            for (int c = lane; c < a.dv; c += 32) kv_store<KT>(dst + c, src[c]);
        }
    }
}

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAXC = 8;      // value columns per lane: dv <= 256

// Block = (row, head, split); its warps walk 32-key tiles of the split's key range, one key per lane for the scores, one value
// column set per lane for the weighted sum, online softmax per warp; warps, then splits, merge in a fixed order.
template <typename KT>
__global__ void __launch_bounds__(ATT_WARPS * 32) sink_attention_kernel(RaggedBatch rb, SinkAttnArgs a) {
    extern __shared__ float smem[];
    float* sq = smem;                                   // [d]
    float* sm = sq + a.d;                               // [ATT_WARPS] m, [ATT_WARPS] l, [ATT_WARPS, dv] acc
    const int r = blockIdx.x, h = blockIdx.y, sp = blockIdx.z, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = rb.row_entry[r], pos = rb.row_pos[r], slot = rb.ent_slot[e];
    const int g = h / (a.H / a.G), d = a.d, dv = a.dv;
    const int* bt = a.block_table + (size_t)slot * a.max_pages;
    for (int c = threadIdx.x; c < d; c += blockDim.x) sq[c] = a.q[(size_t)r * a.ldq + (size_t)h * d + c] * a.scale;
    __syncthreads();
    const int nkeys = pos + 1;
    const int ntiles = (nkeys + 31) / 32, per = (ntiles + a.nsplit - 1) / a.nsplit;
    const int t_lo = sp * per, t_hi = min(ntiles, t_lo + per);
    float m = -INFINITY, l = 0.f, acc[ATT_MAXC];
#pragma unroll
    for (int c = 0; c < ATT_MAXC; ++c) acc[c] = 0.f;
    const bool vec = (d & 3) == 0 && sizeof(KT) == 4;
    for (int t = t_lo + warp; t < t_hi; t += ATT_WARPS) {
        const int j = t * 32 + lane;
        const int pg = bt[(t * 32) / KV_PAGE];           // a 32-key tile never straddles a 64-token page
        const size_t base = ((size_t)pg * a.G + g) * KV_PAGE + ((t * 32) % KV_PAGE);
        float s = -INFINITY;
        if (j < nkeys) {
            const KT* kr = (const KT*)a.k_pool + (base + lane) * d;
            float dot = 0.f;
            if (vec) {
                const float4* k4 = reinterpret_cast<const float4*>(kr);
                for (int c = 0; c < d / 4; ++c) {
                    const float4 kk = k4[c];
                    dot = fmaf(sq[4 * c], kk.x, dot); dot = fmaf(sq[4 * c + 1], kk.y, dot);
                    dot = fmaf(sq[4 * c + 2], kk.z, dot); dot = fmaf(sq[4 * c + 3], kk.w, dot);
                }
            } else {
                for (int c = 0; c < d; ++c) dot = fmaf(sq[c], kv_load<KT>(kr + c), dot);
            }
            s = dot;
        }
        const float tm = warp_max(s);
        const float mn = fmaxf(m, tm);
        const float corr = (m == -INFINITY) ? 0.f : __expf(m - mn);
        const float p = (j < nkeys) ? __expf(s - mn) : 0.f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int c = 0; c < ATT_MAXC; ++c) acc[c] *= corr;
        m = mn;
        const int cnt = min(32, nkeys - t * 32);
        const KT* vb = (const KT*)a.v_pool + base * dv;
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
#pragma unroll
            for (int c = 0; c < ATT_MAXC; ++c) {
                const int col = lane + 32 * c;
                if (col < dv) acc[c] = fmaf(pj, kv_load<KT>(vb + (size_t)jj * dv + col), acc[c]);
            }
        }
    }
    // merge the warps in warp order
    float* wm = sm; float* wl = sm + ATT_WARPS; float* wa = sm + 2 * ATT_WARPS;
    if (lane == 0) { wm[warp] = m; wl[warp] = l; }
#pragma unroll
    for (int c = 0; c < ATT_MAXC; ++c) { const int col = lane + 32 * c; if (col < dv) wa[warp * dv + col] = acc[c]; }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, wm[w]);
    const bool last = a.nsplit == 1;
    const float sink = (last && a.sink) ? a.sink[h] : -INFINITY;
    const float Mx = fmaxf(M, sink);
    float Lsum = (sink == -INFINITY) ? 0.f : __expf(sink - Mx);
    float wsc[ATT_WARPS];
    for (int w = 0; w < ATT_WARPS; ++w) { wsc[w] = (wm[w] == -INFINITY) ? 0.f : __expf(wm[w] - Mx); Lsum += wl[w] * wsc[w]; }
    for (int col = threadIdx.x; col < dv; col += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < ATT_WARPS; ++w) o += wa[w * dv + col] * wsc[w];
        if (last) store_act(a.out, r, h * dv + col, o / Lsum);
        else a.part[(((size_t)r * a.H + h) * a.nsplit + sp) * (dv + 2) + 2 + col] = o;
    }
    if (!last && threadIdx.x == 0) {
        float* pp = a.part + (((size_t)r * a.H + h) * a.nsplit + sp) * (dv + 2);
        pp[0] = Mx; pp[1] = Lsum;          // (no sink yet: Mx == M, possibly -inf for an empty split)
    }
}

__global__ void sink_attention_merge_kernel(SinkAttnArgs a) {
    const int r = blockIdx.x, h = blockIdx.y, dv = a.dv;
    const float* pp = a.part + ((size_t)r * a.H + h) * a.nsplit * (dv + 2);
    const float sink = a.sink ? a.sink[h] : -INFINITY;
    float Mx = sink;
    for (int s = 0; s < a.nsplit; ++s) Mx = fmaxf(Mx, pp[(size_t)s * (dv + 2)]);
    float L = (sink == -INFINITY) ? 0.f : __expf(sink - Mx);
    for (int s = 0; s < a.nsplit; ++s) {
        const float ms = pp[(size_t)s * (dv + 2)];
        if (ms != -INFINITY) L += pp[(size_t)s * (dv + 2) + 1] * __expf(ms - Mx);
    }
    for (int col = threadIdx.x; col < dv; col += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < a.nsplit; ++s) {
            const float ms = pp[(size_t)s * (dv + 2)];
            if (ms != -INFINITY) o += pp[(size_t)s * (dv + 2) + 2 + col] * __expf(ms - Mx);
        }
        store_act(a.out, r, h * dv + col, o / L);
    }
}

// ---------------------------------------------------------------------------------------------------------------- Mamba-2
// Causal depthwise convolution over the x | B | C columns + SiLU.  The taps that reach before the entry's first row read the
// sequence's carried window (zeros for a new sequence).
__global__ void conv_silu_kernel(RaggedBatch rb, Mamba2Args a, int C, int col0) {
    const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int e = rb.row_entry[r], i = r - rb.ent_row0[e], slot = rb.ent_slot[e], taps = a.taps;
    const float* win = a.conv_state + (size_t)slot * (taps - 1) * C;
    float acc = a.conv_b[c];
    for (int k = 0; k < taps; ++k) {
        const int back = taps - 1 - k;                   // this tap reads the input `back` tokens ago
        const float u = (i - back >= 0) ? a.proj[(size_t)(r - back) * a.ldp + col0 + c] : win[(size_t)(taps - 1 + i - back) * C + c];
        acc = fmaf(a.conv_w[(size_t)c * taps + k], u, acc);
    }
    a.xbc[(size_t)r * C + c] = acc / (1.f + __expf(-acc));
}
// New window = the last taps-1 inputs of the sequence (older ones shift down when the entry is shorter than the window).
__global__ void conv_window_kernel(RaggedBatch rb, Mamba2Args a, int C, int col0) {
    const int e = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int len = rb.ent_len[e], r0 = rb.ent_row0[e], slot = rb.ent_slot[e], nwin = a.taps - 1;
    float* win = a.conv_state + (size_t)slot * nwin * C;
    for (int i = 0; i < nwin; ++i) {
        const int src = len - nwin + i;                  // index among this entry's rows
        win[(size_t)i * C + c] = (src >= 0) ? a.proj[(size_t)(r0 + src) * a.ldp + col0 + c] : win[(size_t)(i + len) * C + c];
    }
}

// Selective scan, one block per (entry, head, 128-column slice of P); thread (p, ns) owns state rows n = ns, ns + 8, ...
constexpr int SSD_NS = 8, SSD_MAXR = 32;      // N <= 256
__global__ void ssd_scan_kernel(RaggedBatch rb, Mamba2Args a, int C) {
    const int e = blockIdx.x, h = blockIdx.y, ns = threadIdx.x & (SSD_NS - 1), pl = threadIdx.x / SSD_NS;
    const int p = blockIdx.z * (blockDim.x / SSD_NS) + pl;
    const int P = a.P, N = a.N, inner = a.heads * P, g = h / (a.heads / a.groups);
    const bool live = p < P;
    const int len = rb.ent_len[e], r0 = rb.ent_row0[e], slot = rb.ent_slot[e];
    float* S = a.ssm_state + (((size_t)slot * a.heads + h) * N) * P;
    float s[SSD_MAXR];
    const int nr = (N + SSD_NS - 1) / SSD_NS;
#pragma unroll
    for (int i = 0; i < SSD_MAXR; ++i) { const int n = ns + SSD_NS * i; s[i] = (i < nr && n < N && live) ? S[(size_t)n * P + p] : 0.f; }
    const float negA = -__expf(a.A_log[h]), Dh = a.D[h], dtb = a.dt_bias[h];
    const int dtcol = 2 * inner + 2 * a.groups * N + h;
    for (int t = 0; t < len; ++t) {
        const int r = r0 + t;
        const float z = a.proj[(size_t)r * a.ldp + dtcol] + dtb;
        const float dt = (z > 20.f) ? z : log1pf(__expf(z));
        const float decay = __expf(negA * dt);
        const float* xr = a.xbc + (size_t)r * C;
        const float xv = live ? xr[h * P + p] : 0.f;
        const float* Br = xr + inner + g * N;
        const float* Cr = Br + a.groups * N;
        const float dx = dt * xv;
        float y = 0.f;
#pragma unroll
        for (int i = 0; i < SSD_MAXR; ++i) {
            const int n = ns + SSD_NS * i;
            if (i < nr && n < N) {
                s[i] = fmaf(decay, s[i], Br[n] * dx);
                y = fmaf(s[i], Cr[n], y);
            }
        }
#pragma unroll
        for (int o = SSD_NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        if (ns == 0 && live) a.y[(size_t)r * inner + h * P + p] = y + Dh * xv;
    }
#pragma unroll
    for (int i = 0; i < SSD_MAXR; ++i) { const int n = ns + SSD_NS * i; if (i < nr && n < N && live) S[(size_t)n * P + p] = s[i]; }
}

// out = unit_rms_per_group(y * silu(z)) * w : block per (row, group)
__global__ void gated_group_rms_kernel(Mamba2Args a) {
    __shared__ float scratch[32];
    const int r = blockIdx.x, gi = blockIdx.y, inner = a.heads * a.P, gs = inner / a.norm_groups;
    const float* y = a.y + (size_t)r * inner + gi * gs;
    const float* z = a.proj + (size_t)r * a.ldp + gi * gs;
    float ss = 0.f;
    for (int c = threadIdx.x; c < gs; c += blockDim.x) { const float zz = z[c], v = y[c] * (zz / (1.f + __expf(-zz))); ss += v * v; }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)gs + a.eps);
    for (int c = threadIdx.x; c < gs; c += blockDim.x) {
        const float zz = z[c], v = y[c] * (zz / (1.f + __expf(-zz)));
        store_act(a.out, r, gi * gs + c, v * inv * a.norm_w[gi * gs + c]);
    }
}

// ---------------------------------------------------------------------------------------------------------------- feed-forwards
__global__ void clamped_glu_kernel(const float* __restrict__ gu, int ld, int up_off, int F, float limit, ActOut out) {
    const int r = blockIdx.y, j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= F) return;
    const float g = fminf(gu[(size_t)r * ld + j], limit);
    const float u = fminf(fmaxf(gu[(size_t)r * ld + up_off + j], -limit), limit);
    store_act(out, r, j, g / (1.f + __expf(-1.702f * g)) * (u + 1.f));
}

// softmax over all experts, the `top` largest (ties: lowest index), weights = the scores themselves.  One warp per row.
__global__ void route_kernel(MoeArgs a) {
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= a.T) return;
    const float* z = a.router_logits + (size_t)r * a.ldr;
    float mx = -INFINITY;
    for (int e = lane; e < a.E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float den = 0.f;
    for (int e = lane; e < a.E; e += 32) den += expf(z[e] - mx);
    den = warp_sum(den);
    unsigned long long taken[4] = {0, 0, 0, 0};         // E <= 256: bit per expert, same in every lane
    for (int k = 0; k < a.top; ++k) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < a.E; e += 32)
            if (!((taken[e >> 6] >> (e & 63)) & 1ull) && (z[e] > bv)) { bv = z[e]; bi = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        taken[bi >> 6] |= 1ull << (bi & 63);
        if (lane == 0) { a.sel_e[(size_t)r * a.top + k] = bi; a.sel_w[(size_t)r * a.top + k] = expf(bv - mx) / den; }
    }
}

// Counting sort of the (row, choice) pairs by expert + the tile map of the grouped linears (32 pairs per tile).  One block.
__global__ void moe_sort_kernel(MoeArgs a) {
    extern __shared__ int sh[];
    int* cnt = sh; int* off = sh + a.E; int* fill = sh + 2 * a.E;
    const int n = a.T * a.top;
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) { cnt[e] = 0; fill[e] = 0; }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[a.sel_e[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, t = 0;
        for (int e = 0; e < a.E; ++e) {
            off[e] = o;
            for (int r0 = 0; r0 < cnt[e]; r0 += 32) { a.tile_e[t] = e; a.tile_r0[t] = o + r0; a.tile_n[t] = min(32, cnt[e] - r0); ++t; }
            o += cnt[e];
        }
        *a.n_tiles = t;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const int e = a.sel_e[i]; a.sorted[off[e] + atomicAdd(&fill[e], 1)] = i; }
}

// Grouped linear: tile = 32 pairs of one expert x 64 output columns.  UP: act[pair] = gelu_erf(up_e h[row of pair]); else y[pair] = down_e act[pair].
template <bool UP>
__global__ void __launch_bounds__(256) moe_linear_kernel(MoeArgs a) {
    __shared__ float sa[16][32 + 1], sw[16][64 + 4];
    __shared__ int spair[32];
    const int tile = blockIdx.y;
    if (tile >= *a.n_tiles) return;
    const int e = a.tile_e[tile], r0 = a.tile_r0[tile], nr = a.tile_n[tile];
    const int N = UP ? a.F : a.W, K = UP ? a.W : a.F, ldw = UP ? a.ldwu : a.ldwd;
    const bf16* Wt = UP ? a.up[e] : a.down[e];
    const int n0 = blockIdx.x * 64, tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;      // thread: 2 pairs x 4 columns
    if (tid < 32) spair[tid] = tid < nr ? a.sorted[r0 + tid] : -1;
    __syncthreads();
    float acc[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = tid; i < 32 * 16; i += 256) {
            const int r = i >> 4, k = i & 15, pr = spair[r];
            float v = 0.f;
            if (pr >= 0 && k0 + k < K) v = UP ? a.h[(size_t)(pr / a.top) * a.ldh + k0 + k] : a.act[(size_t)pr * a.lda + k0 + k];
            sa[k][r] = v;
        }
        for (int i = tid; i < 64 * 16; i += 256) {
            const int r = i >> 4, k = i & 15;
            sw[k][r] = (n0 + r < N && k0 + k < K) ? __bfloat162float(Wt[(size_t)(n0 + r) * ldw + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float a0 = sa[k][ty * 2], a1 = sa[k][ty * 2 + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float w = sw[k][tx * 4 + j]; acc[0][j] = fmaf(a0, w, acc[0][j]); acc[1][j] = fmaf(a1, w, acc[1][j]); }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int pr = spair[ty * 2 + i];
        if (pr < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (UP) a.act[(size_t)pr * a.lda + n] = gelu_erf_f(acc[i][j]);
            else a.y[(size_t)pr * a.ldy + n] = acc[i][j];
        }
    }
}

__global__ void moe_combine_kernel(MoeArgs a) {
    const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.W) return;
    float s = 0.f;
    for (int k = 0; k < a.top; ++k) s = fmaf(a.sel_w[(size_t)r * a.top + k], a.y[((size_t)r * a.top + k) * a.ldy + c], s);
    a.x[(size_t)r * a.ldx + c] += s;
}

inline int last_err() { return (int)cudaGetLastError(); }

}  // namespace

// ---------------------------------------------------------------------------------------------------------------- launchers
int embed_scale_rows_launch(cudaStream_t st, const int* ids, int T, const bf16* embed, int W, float scale, float* x, int ldx) {
    embed_scale_rows_kernel<<<T, 128, 0, st>>>(ids, T, embed, W, scale, x, ldx);
    return last_err();
}
int dyt_rows_launch(cudaStream_t st, const float* x, int ldx, const int* rows, int R, int W, const float* alpha, const float* w, const float* b,
                    const ActOut& out) {
    dyt_rows_kernel<<<R, 128, 0, st>>>(x, ldx, rows, W, alpha, w, b, out);
    return last_err();
}
int gather_rows_launch(cudaStream_t st, const float* src, int lds, const int* rows, int R, int W, float* dst, int ldd) {
    gather_rows_kernel<<<R, 128, 0, st>>>(src, lds, rows, W, dst, ldd);
    return last_err();
}
int linear_f32_launch(cudaStream_t st, const float* A, int lda, const bf16* W, int ldw, int M, int N, int K, int mode, float* C, int ldc) {
    if (M <= 0 || N <= 0 || K <= 0) return -1000;
    const dim3 grid((N + 63) / 64, (M + 63) / 64);
    if (mode == LIN_RESID) linear_f32_kernel<LIN_RESID><<<grid, 256, 0, st>>>(A, lda, W, ldw, M, N, K, C, ldc);
    else linear_f32_kernel<LIN_STORE><<<grid, 256, 0, st>>>(A, lda, W, ldw, M, N, K, C, ldc);
    return last_err();
}
int attn_prep_launch(cudaStream_t st, const RaggedBatch& rb, const AttnPrepArgs& a) {
    if (a.kv_f32) attn_prep_kernel<float><<<rb.T, 256, 0, st>>>(rb, a);
    else attn_prep_kernel<bf16><<<rb.T, 256, 0, st>>>(rb, a);
    return last_err();
}
int sink_attention_launch(cudaStream_t st, const RaggedBatch& rb, const SinkAttnArgs& a) {
    if (a.dv > 32 * ATT_MAXC || a.H % a.G) return -1000;
    const size_t smem = (size_t)(a.d + 2 * ATT_WARPS + ATT_WARPS * a.dv) * sizeof(float);
    const dim3 grid(rb.T, a.H, a.nsplit);
    if (a.kv_f32) sink_attention_kernel<float><<<grid, ATT_WARPS * 32, smem, st>>>(rb, a);
    else sink_attention_kernel<bf16><<<grid, ATT_WARPS * 32, smem, st>>>(rb, a);
    int e = last_err();
    if (e || a.nsplit == 1) return e;
    sink_attention_merge_kernel<<<dim3(rb.T, a.H), 64, 0, st>>>(a);
    return last_err();
}
int mamba2_launch_count() { return 4; }
int mamba2_mixer_launch(cudaStream_t st, const RaggedBatch& rb, const Mamba2Args& a) {
    const int inner = a.heads * a.P, C = inner + 2 * a.groups * a.N;
    if (a.N > SSD_NS * SSD_MAXR || a.heads % a.groups || inner % a.norm_groups || a.taps < 1) return -1000;
    conv_silu_kernel<<<dim3((C + 127) / 128, rb.T), 128, 0, st>>>(rb, a, C, inner);
    int e = last_err();
    if (e) return e;
    if (a.taps > 1) {
        conv_window_kernel<<<dim3((C + 127) / 128, rb.E), 128, 0, st>>>(rb, a, C, inner);
        if ((e = last_err())) return e;
    }
    const int pcols = a.P < 128 ? a.P : 128;
    ssd_scan_kernel<<<dim3(rb.E, a.heads, (a.P + pcols - 1) / pcols), pcols * SSD_NS, 0, st>>>(rb, a, C);
    if ((e = last_err())) return e;
    gated_group_rms_kernel<<<dim3(rb.T, a.norm_groups), 128, 0, st>>>(a);
    return last_err();
}
int clamped_glu_launch(cudaStream_t st, const float* gu, int ld, int up_off, int T, int F, float limit, const ActOut& out) {
    clamped_glu_kernel<<<dim3((F + 127) / 128, T), 128, 0, st>>>(gu, ld, up_off, F, limit, out);
    return last_err();
}
int moe_launch(cudaStream_t st, const MoeArgs& a) {
    if (a.E > 256 || a.top > a.E || a.top < 1) return -1000;
    route_kernel<<<(a.T + 3) / 4, 128, 0, st>>>(a);
    int e = last_err();
    if (e) return e;
    moe_sort_kernel<<<1, 1024, (size_t)3 * a.E * sizeof(int), st>>>(a);
    if ((e = last_err())) return e;
    moe_linear_kernel<true><<<dim3((a.F + 63) / 64, a.max_tiles), 256, 0, st>>>(a);
    if ((e = last_err())) return e;
    moe_linear_kernel<false><<<dim3((a.W + 63) / 64, a.max_tiles), 256, 0, st>>>(a);
    if ((e = last_err())) return e;
    moe_combine_kernel<<<dim3((a.W + 127) / 128, a.T), 128, 0, st>>>(a);
    return last_err();
}

}  // namespace cb
