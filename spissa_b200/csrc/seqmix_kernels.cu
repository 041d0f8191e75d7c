// Sequence mixers beyond softmax attention over one map, with the small kernels that surround them.
//
//   dyt_norm          y = tanh(alpha·x) ⊙ w + b                 (a norm without statistics)
//   token_shift       h_t ← h_t + (h_{t-1} − h_t) ⊙ mu          (h_{-1} = 0; the last h is a sequence's state)
//   diff_qkv_store    bias, rotation of interleaved pairs on the first dims of every sub-head, q out, k / v to pages
//   diff_attention    two softmax maps per head over one set of values, combined as a1 − λ·a2, unit rms per head;
//                     scores capped by c·tanh(s/c); a sliding window that also keeps the first tokens
//   retention         S_t = γ_h S_{t-1} + k_t v_tᵀ, o_t = S_tᵀ q_t, unit rms per head, gate silu(g)
//   mingru            S_t = (1 − z_t) S_{t-1} + z_t c_t element by element, gate silu(g)
//   polynorm          a·N(z) + b·N(z²) + c·N(z³) + e with N(v) = v / rms(v) over a token's row
//   add_bias          rows of a 32-bit matrix += a vector
//
// Everything here is computed in 32-bit from 32-bit projections (FFMA, expf / tanhf / sqrtf / division without
// fast-math); only the stores round to the activation type. States are 32-bit. Every output row is reduced in an
// order that depends on its own sequence only, never on the batch or on how the tokens were cut into steps beyond
// the point where a step begins (a recurrence restarts from the stored state, which is exact).
#include "common.cuh"

SP_API const char* sp_seqmix_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(seqmix)

__device__ __forceinline__ float sm_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float sm_silu(float x) { return x / (1.0f + expf(-x)); }

// ============================================================== dynamic tanh norm
// One block per output row; ``rows`` (optional) gathers input rows.
__global__ void dyt_norm_kernel(const float* __restrict__ x, const void* __restrict__ w, const void* __restrict__ b,
                                const void* __restrict__ alpha, int w_dt, void* __restrict__ out, int out_dt,
                                const int* __restrict__ rows, int n_rows, int H) {
    const int r = blockIdx.x;
    if (r >= n_rows) return;
    const float a = sp_ld_dt(alpha, w_dt, 0);
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        sp_st_dt(out, out_dt, (size_t)r * H + c, tanhf(a * x[src + c]) * sp_ld_dt(w, w_dt, c) + sp_ld_dt(b, w_dt, c));
}

SP_API int sp_dyt_norm(const float* x, const void* w, const void* b, const void* alpha, int w_dt, void* out, int out_dt,
                       const int* rows, int n_rows, int H, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    dyt_norm_kernel<<<n_rows, H >= 1024 ? 256 : 128, 0, stream>>>(x, w, b, alpha, w_dt, out, out_dt, rows, n_rows, H);
    SP_CHECK_LAUNCH("dyt_norm");
    return 0;
}

// ============================================================== token shift (with the norm in front of it, if it is dyt)
// DYT: ``x`` is the 32-bit residual stream and h = dyt(x); else ``x`` holds h itself in ``x_dt``.
// A token that is the first of its sequence in this step takes h_{t-1} from state[slot] (zero for a new sequence).
// ``save``: 1 = the block of a sequence's last token also stores its h as the new state. That is only safe when no
// other block reads that row, i.e. when every sequence brings one token; otherwise the host launches the save kernel
// behind this one.
struct ShiftArgs {
    const void* x; int x_dt;
    const void* w; const void* b; const void* alpha; int w_dt;      // dyt (unused when !DYT)
    const void* mu; int mu_dt;
    float* state;                                                    // [slots][H]
    void* out; int out_dt;
    const int* token_seq; const int* seq_start; const int* seq_slot;
    int T, H, n_slots;
};

template <bool DYT>
__device__ __forceinline__ float shift_h(const ShiftArgs& a, size_t row, int c, float alpha) {
    if (DYT) return tanhf(alpha * ((const float*)a.x)[row * a.H + c]) * sp_ld_dt(a.w, a.w_dt, c) + sp_ld_dt(a.b, a.w_dt, c);
    return sp_ld_dt(a.x, a.x_dt, row * a.H + c);
}

template <bool DYT>
__global__ void token_shift_kernel(ShiftArgs a, int save) {
    const int t = blockIdx.x;
    if (t >= a.T) return;
    const int s = a.token_seq[t];
    const bool first = t == a.seq_start[s], last = t + 1 == a.seq_start[s + 1];
    const int slot = a.seq_slot[s];
    if (slot < 0 || slot >= a.n_slots) return;
    const float alpha = DYT ? sp_ld_dt(a.alpha, a.w_dt, 0) : 0.0f;
    float* st = a.state + (size_t)slot * a.H;
    for (int c = threadIdx.x; c < a.H; c += blockDim.x) {
        const float h = shift_h<DYT>(a, t, c, alpha);
        const float prev = first ? st[c] : shift_h<DYT>(a, t - 1, c, alpha);
        sp_st_dt(a.out, a.out_dt, (size_t)t * a.H + c, h + (prev - h) * sp_ld_dt(a.mu, a.mu_dt, c));
        if (save && last) st[c] = h;
    }
}

// Dynamic tanh + shift for widths that are multiples of four: a block takes TS_ROWS neighbouring tokens and a thread
// four neighbouring columns (16-byte loads of the stream and of the state); a token's h serves as the next token's
// "previous" without being computed again, so a row costs 1 + 1/rows tanh per element instead of two. The state
// needs no second launch: see the comment at the store.
#define TS_ROWS 4              // for steps of many tokens; a step of few tokens gives every token a block of its own
__global__ void dyt_shift_rows_kernel(ShiftArgs a, int rows) {
    const int t0 = blockIdx.x * rows;
    const float alpha = sp_ld_dt(a.alpha, a.w_dt, 0);
    const float* x = (const float*)a.x;
    for (int c = threadIdx.x * 4; c < a.H; c += blockDim.x * 4) {
        float w[4], b[4], mu[4], hp[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w[i] = sp_ld_dt(a.w, a.w_dt, c + i);
            b[i] = sp_ld_dt(a.b, a.w_dt, c + i);
            mu[i] = sp_ld_dt(a.mu, a.mu_dt, c + i);
        }
        for (int r = 0; r < rows && t0 + r < a.T; ++r) {
            const int t = t0 + r;
            const int s = a.token_seq[t];
            const bool first = t == a.seq_start[s];
            const int slot = a.seq_slot[s];
            if (slot < 0 || slot >= a.n_slots) continue;
            float* st = a.state + (size_t)slot * a.H + c;
            const float4 cur = *(const float4*)(x + (size_t)t * a.H + c);
            const float xc[4] = {cur.x, cur.y, cur.z, cur.w};
            float h[4], prev[4], o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = tanhf(alpha * xc[i]) * w[i] + b[i];
            if (first) {
                const float4 p4 = *(const float4*)st;
                prev[0] = p4.x; prev[1] = p4.y; prev[2] = p4.z; prev[3] = p4.w;
                // this thread is the only reader of the row in this step, so it is also the one that may overwrite it:
                // with the h of the sequence's last token of the step
                const int t_last = a.seq_start[s + 1] - 1;
                if (t_last == t) {
                    *(float4*)st = make_float4(h[0], h[1], h[2], h[3]);
                } else {
                    const float4 l4 = *(const float4*)(x + (size_t)t_last * a.H + c);
                    *(float4*)st = make_float4(tanhf(alpha * l4.x) * w[0] + b[0], tanhf(alpha * l4.y) * w[1] + b[1],
                                               tanhf(alpha * l4.z) * w[2] + b[2], tanhf(alpha * l4.w) * w[3] + b[3]);
                }
            } else if (r == 0) {
                const float4 p4 = *(const float4*)(x + (size_t)(t - 1) * a.H + c);
                const float xo[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) prev[i] = tanhf(alpha * xo[i]) * w[i] + b[i];
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) prev[i] = hp[i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) { o[i] = h[i] + (prev[i] - h[i]) * mu[i]; hp[i] = h[i]; }
            if (a.out_dt == SP_DT_F32) *(float4*)((float*)a.out + (size_t)t * a.H + c) = make_float4(o[0], o[1], o[2], o[3]);
            else {
                __nv_bfloat162 p0 = __floats2bfloat162_rn(o[0], o[1]), p1 = __floats2bfloat162_rn(o[2], o[3]);
                uint2 pk;
                pk.x = *(uint32_t*)&p0; pk.y = *(uint32_t*)&p1;
                *(uint2*)((__nv_bfloat16*)a.out + (size_t)t * a.H + c) = pk;
            }
        }
    }
}

template <bool DYT>
__global__ void token_shift_save_kernel(ShiftArgs a, int B) {
    const int s = blockIdx.x;
    if (s >= B) return;
    const int slot = a.seq_slot[s];
    if (slot < 0 || slot >= a.n_slots) return;
    const int t = a.seq_start[s + 1] - 1;
    if (t < a.seq_start[s]) return;
    const float alpha = DYT ? sp_ld_dt(a.alpha, a.w_dt, 0) : 0.0f;
    for (int c = threadIdx.x; c < a.H; c += blockDim.x) a.state[(size_t)slot * a.H + c] = shift_h<DYT>(a, t, c, alpha);
}

SP_API int sp_token_shift(const void* x, int x_dt, const void* w, const void* b, const void* alpha, int w_dt,
                          const void* mu, int mu_dt, float* state, int n_slots, void* out, int out_dt,
                          const int* token_seq, const int* seq_start, const int* seq_slot, int T, int B, int H,
                          int all_single, cudaStream_t stream) {
    if (T <= 0) return 0;
    const bool dyt = w != nullptr;
    if (dyt && x_dt != SP_DT_F32) SP_FAIL("token_shift: the norm reads the 32-bit residual stream");
    ShiftArgs a{x, x_dt, w, b, alpha, w_dt, mu, mu_dt, state, out, out_dt, token_seq, seq_start, seq_slot, T, H, n_slots};
    const int threads = H >= 1024 ? 256 : 128;
    if (dyt && (H & 3) == 0 && ((((uintptr_t)x) | ((uintptr_t)state) | ((uintptr_t)out)) & 15) == 0) {
        const int rows = T >= 256 ? TS_ROWS : 1;
        dyt_shift_rows_kernel<<<(T + rows - 1) / rows, H >= 2048 ? 256 : 128, 0, stream>>>(a, rows);
        SP_CHECK_LAUNCH("dyt_shift_rows");
        return 0;                                      // this kernel stores the state itself
    }
    if (dyt) token_shift_kernel<true><<<T, threads, 0, stream>>>(a, all_single);
    else token_shift_kernel<false><<<T, threads, 0, stream>>>(a, all_single);
    SP_CHECK_LAUNCH("token_shift");
    if (!all_single) {
        if (dyt) token_shift_save_kernel<true><<<B, threads, 0, stream>>>(a, B);
        else token_shift_save_kernel<false><<<B, threads, 0, stream>>>(a, B);
        SP_CHECK_LAUNCH("token_shift_save");
    }
    return 0;
}

// ============================================================== where a token's keys and values live
struct KvPlace {
    const int* token_seq;     // [T] sequence index of each token
    const int* positions;     // [T] absolute position of each token
    const int* seq_slot;      // [B] row of each sequence in the page table
    const int* page_table;    // [rows][max_pages]
    int max_pages;
    int page_size;
    SpRange rg;
};

__device__ __forceinline__ bool kv_page_of(const KvPlace& pl, int t, int pos, int& page) {
    const int row = pl.seq_slot[pl.token_seq[t]];
    if (!sp_index_ok(row, pl.rg.n_rows, pl.rg, 402) || !sp_index_ok(pos / pl.page_size, pl.max_pages, pl.rg, 403)) return false;
    page = pl.page_table[(size_t)row * pl.max_pages + pos / pl.page_size];
    return sp_index_ok(page, pl.rg.n_pages, pl.rg, 401);
}

// ============================================================== bias + rotation of interleaved pairs + cache write
// A row of ``qkv`` (32-bit) is [nq sub-heads of d | nk sub-heads of d | G value heads of vd]. A sub-head is one
// map of one head; the first ``rd`` dims of each are rotated, dim 2i with dim 2i+1 by the angle position·inv_freq[i].
// q goes to ``q_out`` [T][nq·d]; the k sub-heads of kv head g are the contiguous row of 2·d (nk/G · d) numbers that
// the key pool holds for the token, [page][G][page_size][nk/G·d]; v likewise with rows of vd.
template <typename TO, typename TC>
__global__ void diff_qkv_store_kernel(const float* __restrict__ qkv, const void* __restrict__ bias, int b_dt,
                                      TO* __restrict__ q_out, TC* __restrict__ kpool, TC* __restrict__ vpool, KvPlace pl,
                                      const float* __restrict__ inv_freq, int T, int nq, int nk, int G, int d, int vd,
                                      int rd, float* __restrict__ stream, const void* __restrict__ stream_bias, int width) {
    extern __shared__ float cs[];                  // [2][rd/2]
    const int t = blockIdx.x;
    if (t >= T) return;
    // the output projection's bias goes into the token's row of the residual stream here, ahead of the product that
    // accumulates into it: one launch less than adding it behind
    if (stream)
        for (int c = threadIdx.x; c < width; c += blockDim.x) stream[(size_t)t * width + c] += sp_ld_dt(stream_bias, b_dt, c);
    const int pos = pl.positions[t];
    const int half = rd >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * inv_freq[i];
        cs[i] = cosf(ang);
        cs[half + i] = sinf(ang);
    }
    __syncthreads();
    int page = 0;
    const bool place_ok = kv_page_of(pl, t, pos, page);
    const int off = pos % pl.page_size;
    const int row = (nq + nk) * d + G * vd;
    const float* src = qkv + (size_t)t * row;
    const int dp = d >> 1;                          // pairs per sub-head
    const int kd = (nk / G) * d;                    // a key row of one kv head
    if (d & 1) {
        // an odd sub-head size: element by element (two-element stores would not be aligned); the last dim never turns
        for (int e = threadIdx.x; e < (nq + nk) * d; e += blockDim.x) {
            const int sh = e / d, i = e - sh * d;
            float val = src[e] + (bias ? sp_ld_dt(bias, b_dt, e) : 0.0f);
            if (i < rd) {
                const int im = i ^ 1;                                     // the other dim of the pair
                const float other = src[sh * d + im] + (bias ? sp_ld_dt(bias, b_dt, sh * d + im) : 0.0f);
                const float co = cs[i >> 1], si = cs[half + (i >> 1)];
                val = (i & 1) ? val * co + other * si : val * co - other * si;
            }
            if (sh < nq) {
                sp_st(q_out, (size_t)t * nq * d + e, val);
            } else if (place_ok) {
                const int ck = e - nq * d;
                const int g = ck / kd, r = ck - g * kd;
                sp_st(kpool, (((size_t)page * G + g) * pl.page_size + off) * kd + r, val);
            }
        }
    } else
    for (int e = threadIdx.x; e < (nq + nk) * dp; e += blockDim.x) {
        const int sh = e / dp, i = e - sh * dp;
        const int c = sh * d + 2 * i;
        float u = src[c], v = src[c + 1];
        if (bias) { u += sp_ld_dt(bias, b_dt, c); v += sp_ld_dt(bias, b_dt, c + 1); }
        if (2 * i < rd) {
            const float co = cs[i], si = cs[half + i];
            const float ru = u * co - v * si, rv = v * co + u * si;
            u = ru; v = rv;
        }
        if (sh < nq) {
            sp_st2(q_out, (size_t)t * nq * d + c, u, v);
        } else if (place_ok) {
            const int ck = c - nq * d;              // column within the token's key numbers
            const int g = ck / kd, r = ck - g * kd;
            sp_st2(kpool, (((size_t)page * G + g) * pl.page_size + off) * kd + r, u, v);
        }
    }
    if (place_ok) {
        for (int e = threadIdx.x; e < G * vd; e += blockDim.x) {
            const int g = e / vd, r = e - g * vd;
            float v = src[(nq + nk) * d + e];
            if (bias) v += sp_ld_dt(bias, b_dt, (nq + nk) * d + e);
            sp_st(vpool, (((size_t)page * G + g) * pl.page_size + off) * vd + r, v);
        }
    }
}

SP_API int sp_diff_qkv_store(const float* qkv, const void* bias, int b_dt, void* q_out, int q_dt, void* kpool, void* vpool,
                             int cache_dt, const int* token_seq, const int* positions, const int* seq_slot,
                             const int* page_table, int max_pages, int page_size, const float* inv_freq, int T, int nq,
                             int nk, int G, int d, int vd, int rd, float* residual, const void* residual_bias, int width,
                             cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || rd < 0 || rd > d || (rd & 1)) SP_FAIL("qkv_store: the rotated dims %d must be even and at most d %d", rd, d);
    if (G <= 0 || nk % G) SP_FAIL("qkv_store: %d key sub-heads are no multiple of %d kv heads", nk, G);
    if (rd > 0 && !inv_freq) SP_FAIL("qkv_store: a frequency table is needed");
    if (residual && !bias) SP_FAIL("qkv_store: the stream's bias comes with the projections' biases (one storage type)");
    KvPlace pl{token_seq, positions, seq_slot, page_table, max_pages, page_size, sp_range_host};
    const size_t smem = (size_t)rd * sizeof(float);
#define QS_LAUNCH(TO, TC)                                                                                          \
    diff_qkv_store_kernel<TO, TC><<<T, 128, smem, stream>>>(qkv, bias, b_dt, (TO*)q_out, (TC*)kpool, (TC*)vpool, pl, \
                                                           inv_freq, T, nq, nk, G, d, vd, rd, residual, residual_bias, width)
    if (q_dt == SP_DT_F32 && cache_dt == SP_DT_F32) QS_LAUNCH(float, float);
    else if (q_dt == SP_DT_BF16 && cache_dt == SP_DT_BF16) QS_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (q_dt == SP_DT_F32 && cache_dt == SP_DT_BF16) QS_LAUNCH(float, __nv_bfloat16);
    else if (q_dt == SP_DT_BF16 && cache_dt == SP_DT_F32) QS_LAUNCH(__nv_bfloat16, float);
    else SP_FAIL("qkv_store: unsupported dtype codes %d/%d", q_dt, cache_dt);
#undef QS_LAUNCH
    SP_CHECK_LAUNCH("diff_qkv_store");
    return 0;
}

// ============================================================== differential attention over the cache
// One warp per (token, head), both maps at once: lane j scores key j against the head's two query halves, two online
// softmaxes run side by side in 32-bit, and every value row is fetched once for both. A query at position p sees the
// keys max(0, p−window+1) … p (all keys when window = 0) and, before them, the keys 0 … keep_first−1; the visible keys are
// walked as one list, kept ones first. SPLIT: the four warps of a CTA share one (token, head) and take chunks of 32
// keys in turn; warp 0 merges their parts in warp order.
#define DA_WARPS 4
#define DA_MAX_D 128           // per-map query/key size
#define DA_MAX_VD 256          // value size

struct DiffArgs {
    int T, H, G, d, vd, window, keep_first;
    float scale, softcap, lam, eps, out_scale;
};

template <typename TQ, typename TC, bool SPLIT>
__global__ void __launch_bounds__(DA_WARPS * 32)
diff_attention_kernel(const TQ* __restrict__ q, const TC* __restrict__ kpool, const TC* __restrict__ vpool,
                      TQ* __restrict__ out, KvPlace pl, DiffArgs a) {
    __shared__ __align__(16) float qs[DA_WARPS][2 * DA_MAX_D];
    __shared__ float part[SPLIT ? DA_WARPS : 1][2][SPLIT ? DA_MAX_VD : 1];
    __shared__ float part_ml[DA_WARPS][4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long gw = SPLIT ? (long long)blockIdx.x : (long long)blockIdx.x * DA_WARPS + warp;
    if (gw >= (long long)a.T * a.H) return;
    const int t = (int)(gw / a.H), h = (int)(gw % a.H);
    const int g = h / (a.H / a.G);
    const int d = a.d, vd = a.vd, kd = 2 * a.d;
    const int p = pl.positions[t];
    const int row = sp_checked_row(pl.seq_slot[pl.token_seq[t]], pl.rg);
    const int* pt = pl.page_table + (size_t)row * pl.max_pages;
    const int ps = pl.page_size;

    for (int c = lane; c < kd; c += 32) qs[warp][c] = sp_ld(q, ((size_t)t * a.H + h) * kd + c);
    __syncwarp();

    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const int n_first = a.keep_first < lo ? a.keep_first : lo;       // kept keys that lie before the window
    const int n_vis = n_first + (p - lo + 1);
    float m1 = -INFINITY, l1 = 0.0f, m2 = -INFINITY, l2 = 0.0f;
    float acc1[DA_MAX_VD / 32], acc2[DA_MAX_VD / 32];
#pragma unroll
    for (int i = 0; i < DA_MAX_VD / 32; ++i) acc1[i] = acc2[i] = 0.0f;

    for (int v0 = SPLIT ? 32 * warp : 0; v0 < n_vis; v0 += SPLIT ? 32 * DA_WARPS : 32) {
        const int vi = v0 + lane;
        const bool valid = vi < n_vis;
        float s1 = -INFINITY, s2 = -INFINITY;
        int my_page = 0, my_off = 0;
        if (valid) {
            const int j = vi < n_first ? vi : lo + (vi - n_first);
            my_page = sp_checked_page(pt[sp_checked_entry(j / ps, pl.max_pages, pl.rg)], pl.rg);
            my_off = j % ps;
            const TC* kr = kpool + (((size_t)my_page * a.G + g) * ps + my_off) * kd;
            float d1 = 0.0f, d2 = 0.0f;
            for (int c = 0; c < d; ++c) {
                d1 = fmaf(qs[warp][c], sp_ld(kr, c), d1);
                d2 = fmaf(qs[warp][d + c], sp_ld(kr, d + c), d2);
            }
            s1 = d1 * a.scale;
            s2 = d2 * a.scale;
            if (a.softcap > 0.0f) {
                s1 = a.softcap * tanhf(s1 / a.softcap);
                s2 = a.softcap * tanhf(s2 / a.softcap);
            }
        }
        const float n1 = fmaxf(m1, sp_warp_max(s1)), n2 = fmaxf(m2, sp_warp_max(s2));
        const float e1 = valid ? expf(s1 - n1) : 0.0f, e2 = valid ? expf(s2 - n2) : 0.0f;
        const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);            // first chunk: exp(-inf) = 0
        l1 = l1 * c1 + sp_warp_sum(e1);
        l2 = l2 * c2 + sp_warp_sum(e2);
#pragma unroll
        for (int i = 0; i < DA_MAX_VD / 32; ++i) { acc1[i] *= c1; acc2[i] *= c2; }
        const int n_valid = min(32, n_vis - v0);
        for (int jj0 = 0; jj0 < n_valid; jj0 += 4) {
            float w1[4], w2[4];
            const TC* vr[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                w1[u] = __shfl_sync(0xffffffffu, e1, jj0 + u);
                w2[u] = __shfl_sync(0xffffffffu, e2, jj0 + u);
                const int pg = __shfl_sync(0xffffffffu, my_page, jj0 + u);
                const int of = __shfl_sync(0xffffffffu, my_off, jj0 + u);
                vr[u] = vpool + (((size_t)pg * a.G + g) * ps + of) * vd;
            }
#pragma unroll
            for (int i = 0; i < DA_MAX_VD / 32; ++i) {
                const int c = lane + 32 * i;
                if (c < vd) {
                    float v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) v[u] = jj0 + u < n_valid ? sp_ld(vr[u], c) : 0.0f;
#pragma unroll
                    for (int u = 0; u < 4; ++u) { acc1[i] = fmaf(w1[u], v[u], acc1[i]); acc2[i] = fmaf(w2[u], v[u], acc2[i]); }
                }
            }
        }
        m1 = n1;
        m2 = n2;
    }
    if (SPLIT) {
#pragma unroll
        for (int i = 0; i < DA_MAX_VD / 32; ++i) {
            const int c = lane + 32 * i;
            if (c < vd) { part[warp][0][c] = acc1[i]; part[warp][1][c] = acc2[i]; }
        }
        if (lane == 0) { part_ml[warp][0] = m1; part_ml[warp][1] = l1; part_ml[warp][2] = m2; part_ml[warp][3] = l2; }
        __syncthreads();
        if (warp != 0) return;
        float mm1 = -INFINITY, mm2 = -INFINITY;
        for (int w = 0; w < DA_WARPS; ++w) { mm1 = fmaxf(mm1, part_ml[w][0]); mm2 = fmaxf(mm2, part_ml[w][2]); }
        l1 = l2 = 0.0f;
#pragma unroll
        for (int i = 0; i < DA_MAX_VD / 32; ++i) acc1[i] = acc2[i] = 0.0f;
        for (int w = 0; w < DA_WARPS; ++w) {
            if (part_ml[w][1] <= 0.0f) continue;                     // a warp that saw no key
            const float f1 = expf(part_ml[w][0] - mm1), f2 = expf(part_ml[w][2] - mm2);
            l1 += part_ml[w][1] * f1;
            l2 += part_ml[w][3] * f2;
#pragma unroll
            for (int i = 0; i < DA_MAX_VD / 32; ++i) {
                const int c = lane + 32 * i;
                if (c < vd) { acc1[i] = fmaf(part[w][0][c], f1, acc1[i]); acc2[i] = fmaf(part[w][1][c], f2, acc2[i]); }
            }
        }
    }
    // o = a1 − λ·a2, then unit rms over the head's values, then the constant factor
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < DA_MAX_VD / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < vd) {
            acc1[i] = acc1[i] / l1 - a.lam * (acc2[i] / l2);
            ss = fmaf(acc1[i], acc1[i], ss);
        }
    }
    ss = sp_warp_sum(ss);
    const float inv = a.out_scale / sqrtf(ss / (float)vd + a.eps);
#pragma unroll
    for (int i = 0; i < DA_MAX_VD / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < vd) sp_st(out, ((size_t)t * a.H + h) * vd + c, acc1[i] * inv);
    }
}

// The same for steps of few (token, head) pairs over many keys (decoding): eight warps share one pair and take the
// chunks of 32 visible keys in turn; key and value rows are read in 16- and 8-byte pieces (d a multiple of 8, vd of
// 4), a lane owns four neighbouring value columns; warp 0 merges the eight parts in warp order.
#define DD_WARPS 16

__device__ __forceinline__ void dd_ld8(const float* p, float (&v)[8]) {
    const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void dd_ld8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *(const uint4*)p;
    const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
// four neighbouring values as they lie in memory, and their 32-bit values
struct DdRaw4f { float4 r; };
struct DdRaw4h { uint2 r; };
__device__ __forceinline__ void dd_fetch4(const float* p, DdRaw4f& x) { x.r = *(const float4*)p; }
__device__ __forceinline__ void dd_fetch4(const __nv_bfloat16* p, DdRaw4h& x) { x.r = *(const uint2*)p; }
__device__ __forceinline__ void dd_open4(const DdRaw4f& x, float (&v)[4]) { v[0] = x.r.x; v[1] = x.r.y; v[2] = x.r.z; v[3] = x.r.w; }
__device__ __forceinline__ void dd_open4(const DdRaw4h& x, float (&v)[4]) {
    const __nv_bfloat162* h = (const __nv_bfloat162*)&x.r;
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename TC> struct DdRaw { using T = DdRaw4f; static constexpr int BATCH = 8; };
template <> struct DdRaw<__nv_bfloat16> { using T = DdRaw4h; static constexpr int BATCH = 16; };

// Sixteen warps share one (token, head) and take the chunks of 32 visible keys in turn. Per chunk a warp first asks
// for the value rows (a lane owns four neighbouring columns; in bfloat16 sixteen rows of the chunk are in flight at
// once), then reads its keys in 16-byte pieces and computes the two scores, so one memory round trip covers both.
// NV = groups of 128 value columns. Warp 0 merges the parts in warp order.
__device__ __forceinline__ void dd_cp_async16(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dd_cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// ``SR`` key rows of a chunk are staged at a time in the warp's own piece of shared memory by 16-byte asynchronous
// copies in which neighbouring lanes take neighbouring pieces of a row (a lane that read its own row straight from
// global memory touched 32 lines per instruction); each lane then reads its key's row from there.
template <typename TQ, typename TC, int NV>
__global__ void __launch_bounds__(DD_WARPS * 32)
diff_decode_kernel(const TQ* __restrict__ q, const TC* __restrict__ kpool, const TC* __restrict__ vpool,
                   TQ* __restrict__ out, KvPlace pl, DiffArgs a, int SR) {
    using Raw = typename DdRaw<TC>::T;
    constexpr int VB = DdRaw<TC>::BATCH / NV;            // value rows in flight per lane: 16 (bfloat16) or 8, halved for two column groups
    extern __shared__ __align__(16) float dd_sm[];
    float* qs = dd_sm;                                   // [2·d]
    float* part = qs + 2 * a.d;                          // [DD_WARPS][2][vd]
    __shared__ float part_ml[DD_WARPS][4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int g = h / (a.H / a.G);
    const int d = a.d, vd = a.vd, kd = 2 * a.d;
    const int row_pieces = kd * (int)sizeof(TC) / 16;    // 16-byte pieces of a key row
    const int row_stride = kd * (int)sizeof(TC) + 16;    // bytes; the pad spreads the rows over the banks
    uint8_t* kbuf = (uint8_t*)(part + (size_t)DD_WARPS * 2 * vd) + (size_t)warp * SR * row_stride;
    const int p = pl.positions[t];
    const int row = sp_checked_row(pl.seq_slot[pl.token_seq[t]], pl.rg);
    const int* pt = pl.page_table + (size_t)row * pl.max_pages;
    const int ps = pl.page_size;
    for (int c = threadIdx.x; c < kd; c += blockDim.x) qs[c] = sp_ld(q, ((size_t)t * a.H + h) * kd + c);
    __syncthreads();

    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const int n_first = a.keep_first < lo ? a.keep_first : lo;
    const int n_vis = n_first + (p - lo + 1);
    float m1 = -INFINITY, l1 = 0.0f, m2 = -INFINITY, l2 = 0.0f;
    float acc1[NV][4], acc2[NV][4];
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u) acc1[i][u] = acc2[i][u] = 0.0f;

    for (int v0 = 32 * warp; v0 < n_vis; v0 += 32 * DD_WARPS) {
        const int vi = v0 + lane;
        const bool valid = vi < n_vis;
        int my_page = 0, my_off = 0;
        if (valid) {
            const int j = vi < n_first ? vi : lo + (vi - n_first);
            my_page = sp_checked_page(pt[sp_checked_entry(j / ps, pl.max_pages, pl.rg)], pl.rg);
            my_off = j % ps;
        }
        const size_t my_row = ((size_t)my_page * a.G + g) * ps + my_off;     // lanes beyond the end: row 0 of page 0, weight 0
        Raw raw[NV][VB];
        auto fetch = [&](int jj0) {
#pragma unroll
            for (int u = 0; u < VB; ++u) {
                const size_t r = __shfl_sync(0xffffffffu, my_row, (jj0 + u) & 31);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    const int c = 4 * lane + 128 * i;
                    if (c < vd) dd_fetch4(vpool + r * vd + c, raw[i][u]);
                }
            }
        };
        fetch(0);
        float s1 = -INFINITY, s2 = -INFINITY;
        for (int sub = 0; sub * SR < 32; ++sub) {
            const int total = SR * row_pieces;
            for (int e0 = 0; e0 < total; e0 += 32) {
                const int e = e0 + lane;
                const int r = min(e / row_pieces, SR - 1), piece = e % row_pieces;
                const size_t src_row = __shfl_sync(0xffffffffu, my_row, sub * SR + r);
                if (e < total) dd_cp_async16(kbuf + (size_t)r * row_stride + piece * 16, (const uint8_t*)(kpool + src_row * kd) + piece * 16);
            }
            dd_cp_async_wait_all();
            __syncwarp();
            if (valid && lane / SR == sub) {
                const TC* kr = (const TC*)(kbuf + (size_t)(lane % SR) * row_stride);
                float d1 = 0.0f, d2 = 0.0f;
                for (int c = 0; c < d; c += 8) {
                    float k1[8], k2[8];
                    dd_ld8(kr + c, k1);
                    dd_ld8(kr + d + c, k2);
#pragma unroll
                    for (int u = 0; u < 8; ++u) { d1 = fmaf(qs[c + u], k1[u], d1); d2 = fmaf(qs[d + c + u], k2[u], d2); }
                }
                s1 = d1 * a.scale;
                s2 = d2 * a.scale;
                if (a.softcap > 0.0f) {
                    s1 = a.softcap * tanhf(s1 / a.softcap);
                    s2 = a.softcap * tanhf(s2 / a.softcap);
                }
            }
            __syncwarp();
        }
        const float n1 = fmaxf(m1, sp_warp_max(s1)), n2 = fmaxf(m2, sp_warp_max(s2));
        const float e1 = valid ? expf(s1 - n1) : 0.0f, e2 = valid ? expf(s2 - n2) : 0.0f;
        const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);
        l1 = l1 * c1 + sp_warp_sum(e1);
        l2 = l2 * c2 + sp_warp_sum(e2);
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
            for (int u = 0; u < 4; ++u) { acc1[i][u] *= c1; acc2[i][u] *= c2; }
#pragma unroll
        for (int jj0 = 0; jj0 < 32; jj0 += VB) {
            if (jj0 > 0) fetch(jj0);
#pragma unroll
            for (int u = 0; u < VB; ++u) {
                const float w1 = __shfl_sync(0xffffffffu, e1, (jj0 + u) & 31);
                const float w2 = __shfl_sync(0xffffffffu, e2, (jj0 + u) & 31);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    if (4 * lane + 128 * i < vd) {
                        float v[4];
                        dd_open4(raw[i][u], v);
#pragma unroll
                        for (int x = 0; x < 4; ++x) { acc1[i][x] = fmaf(w1, v[x], acc1[i][x]); acc2[i][x] = fmaf(w2, v[x], acc2[i][x]); }
                    }
                }
            }
        }
        m1 = n1;
        m2 = n2;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = 4 * lane + 128 * i;
        if (c < vd) {
            *(float4*)&part[((size_t)warp * 2 + 0) * vd + c] = make_float4(acc1[i][0], acc1[i][1], acc1[i][2], acc1[i][3]);
            *(float4*)&part[((size_t)warp * 2 + 1) * vd + c] = make_float4(acc2[i][0], acc2[i][1], acc2[i][2], acc2[i][3]);
        }
    }
    if (lane == 0) { part_ml[warp][0] = m1; part_ml[warp][1] = l1; part_ml[warp][2] = m2; part_ml[warp][3] = l2; }
    __syncthreads();
    if (warp != 0) return;
    float mm1 = -INFINITY, mm2 = -INFINITY;
    for (int w = 0; w < DD_WARPS; ++w) { mm1 = fmaxf(mm1, part_ml[w][0]); mm2 = fmaxf(mm2, part_ml[w][2]); }
    l1 = l2 = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u) acc1[i][u] = acc2[i][u] = 0.0f;
    for (int w = 0; w < DD_WARPS; ++w) {
        if (part_ml[w][1] <= 0.0f) continue;                     // a warp that saw no key
        const float f1 = expf(part_ml[w][0] - mm1), f2 = expf(part_ml[w][2] - mm2);
        l1 += part_ml[w][1] * f1;
        l2 += part_ml[w][3] * f2;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = 4 * lane + 128 * i;
            if (c < vd) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    acc1[i][u] = fmaf(part[((size_t)w * 2 + 0) * vd + c + u], f1, acc1[i][u]);
                    acc2[i][u] = fmaf(part[((size_t)w * 2 + 1) * vd + c + u], f2, acc2[i][u]);
                }
            }
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = 4 * lane + 128 * i;
        if (c < vd) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                acc1[i][u] = acc1[i][u] / l1 - a.lam * (acc2[i][u] / l2);
                ss = fmaf(acc1[i][u], acc1[i][u], ss);
            }
        }
    }
    ss = sp_warp_sum(ss);
    const float inv = a.out_scale / sqrtf(ss / (float)vd + a.eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = 4 * lane + 128 * i;
        if (c < vd) {
#pragma unroll
            for (int u = 0; u < 4; ++u) sp_st(out, ((size_t)t * a.H + h) * vd + c + u, acc1[i][u] * inv);
        }
    }
}

SP_API int sp_diff_attention(const void* q, int q_dt, const void* kpool, const void* vpool, int cache_dt, void* out,
                             const int* token_seq, const int* positions, const int* seq_slot, const int* page_table,
                             int max_pages, int page_size, int T, int H, int G, int d, int vd, int window, int keep_first,
                             float scale, float softcap, float lam, float eps, float out_scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || d > DA_MAX_D) SP_FAIL("diff_attention: map size %d is beyond this kernel's limit %d", d, DA_MAX_D);
    if (vd <= 0 || vd > DA_MAX_VD) SP_FAIL("diff_attention: value size %d is beyond this kernel's limit %d", vd, DA_MAX_VD);
    if (G <= 0 || H % G) SP_FAIL("diff_attention: %d heads are no multiple of %d kv heads", H, G);
    KvPlace pl{token_seq, positions, seq_slot, page_table, max_pages, page_size, sp_range_host};
    DiffArgs a{T, H, G, d, vd, window, keep_first < 0 ? 0 : keep_first, scale, softcap, lam, eps, out_scale};
    const long long warps = (long long)T * H;
    const bool split = warps <= 2048;
    const long long blocks = split ? warps : (warps + DA_WARPS - 1) / DA_WARPS;
    if (blocks > 2147483647LL) SP_FAIL("diff_attention: too many (token, head) pairs for one launch");
    const size_t esz = cache_dt == SP_DT_F32 ? 4 : 2;
    if (split && d % 8 == 0 && vd % 4 == 0 && (((uintptr_t)kpool | (uintptr_t)vpool) & 15) == 0 && ((size_t)vd * esz) % 8 == 0) {
        // shared memory: the query, the warps' parts, and per warp SR staged key rows (as many as fit 200 KB)
        const size_t dd_fixed = ((size_t)2 * d + (size_t)DD_WARPS * 2 * vd) * sizeof(float);
        const size_t dd_row = (size_t)2 * d * esz + 16;
        int SR = 32;
        while (SR > 1 && dd_fixed + (size_t)DD_WARPS * SR * dd_row > 200 * 1024) SR >>= 1;
        const size_t dd_smem = dd_fixed + (size_t)DD_WARPS * SR * dd_row;
#define DD_LAUNCH(TQ, TC)                                                                                             \
        do {                                                                                                          \
            static SpPerDevice ready;                                                                                 \
            if (!ready.done()) {                                                                                      \
                if (cudaFuncSetAttribute(diff_decode_kernel<TQ, TC, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess || \
                    cudaFuncSetAttribute(diff_decode_kernel<TQ, TC, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)   \
                    SP_FAIL("diff_attention: cannot raise the shared memory limit");                                  \
                ready.mark();                                                                                         \
            }                                                                                                         \
            if (vd <= 128) diff_decode_kernel<TQ, TC, 1><<<(unsigned)blocks, DD_WARPS * 32, dd_smem, stream>>>(       \
                    (const TQ*)q, (const TC*)kpool, (const TC*)vpool, (TQ*)out, pl, a, SR);                           \
            else diff_decode_kernel<TQ, TC, 2><<<(unsigned)blocks, DD_WARPS * 32, dd_smem, stream>>>(                 \
                    (const TQ*)q, (const TC*)kpool, (const TC*)vpool, (TQ*)out, pl, a, SR);                           \
        } while (0)
        if (q_dt == SP_DT_F32 && cache_dt == SP_DT_F32) DD_LAUNCH(float, float);
        else if (q_dt == SP_DT_BF16 && cache_dt == SP_DT_BF16) DD_LAUNCH(__nv_bfloat16, __nv_bfloat16);
        else if (q_dt == SP_DT_F32 && cache_dt == SP_DT_BF16) DD_LAUNCH(float, __nv_bfloat16);
        else if (q_dt == SP_DT_BF16 && cache_dt == SP_DT_F32) DD_LAUNCH(__nv_bfloat16, float);
        else SP_FAIL("diff_attention: unsupported dtype codes %d/%d", q_dt, cache_dt);
#undef DD_LAUNCH
        SP_CHECK_LAUNCH("diff_decode");
        return 0;
    }
#define DA_LAUNCH(TQ, TC)                                                                                             \
    do {                                                                                                              \
        if (split) diff_attention_kernel<TQ, TC, true><<<(unsigned)blocks, DA_WARPS * 32, 0, stream>>>(               \
                (const TQ*)q, (const TC*)kpool, (const TC*)vpool, (TQ*)out, pl, a);                                   \
        else diff_attention_kernel<TQ, TC, false><<<(unsigned)blocks, DA_WARPS * 32, 0, stream>>>(                    \
                (const TQ*)q, (const TC*)kpool, (const TC*)vpool, (TQ*)out, pl, a);                                   \
    } while (0)
    if (q_dt == SP_DT_F32 && cache_dt == SP_DT_F32) DA_LAUNCH(float, float);
    else if (q_dt == SP_DT_BF16 && cache_dt == SP_DT_BF16) DA_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (q_dt == SP_DT_F32 && cache_dt == SP_DT_BF16) DA_LAUNCH(float, __nv_bfloat16);
    else if (q_dt == SP_DT_BF16 && cache_dt == SP_DT_F32) DA_LAUNCH(__nv_bfloat16, float);
    else SP_FAIL("diff_attention: unsupported dtype codes %d/%d", q_dt, cache_dt);
#undef DA_LAUNCH
    SP_CHECK_LAUNCH("diff_attention");
    return 0;
}

// ============================================================== retention, token by token
// proj row (32-bit) = [q: H·d | k: H·d | v: H·vd | g: H·vd]. One CTA per (sequence, head): the state S [d][vd] lives in
// shared memory for the whole step; thread (j, y) owns column j of the rows i ≡ y (mod DY). Per token:
// S ← γ S + (k/√d) vᵀ, o_j = Σ_i S_ij q_i (the DY partial sums added in the order of y), o / rms(o) ⊙ silu(g).
struct RetArgs {
    const float* proj; int ld;
    float* state;                      // [slots][H][d][vd]
    const float* decay;                // [H]
    void* out; int out_dt;             // [T][H·vd]
    const int* seq_start; const int* seq_slot;
    int B, H, d, vd, n_slots;
    float eps;
};

__global__ void retention_scan_kernel(RetArgs a, int vdr, int DY) {
    extern __shared__ float sm[];
    const int d = a.d, vd = a.vd;
    float* S = sm;                         // [d][vd]
    float* qk = S + (size_t)d * vd;        // q [d], k [d]
    float* red = qk + 2 * d;               // [DY][vdr]
    float* o = red + (size_t)DY * vdr;     // [vdr]
    __shared__ float inv_rms;
    const int s = blockIdx.x, h = blockIdx.y;
    const int slot = a.seq_slot[s];
    if (slot < 0 || slot >= a.n_slots) return;
    const int j = threadIdx.x % vdr, y = threadIdx.x / vdr;
    float* gS = a.state + ((size_t)slot * a.H + h) * d * vd;
    for (int e = threadIdx.x; e < d * vd; e += blockDim.x) S[e] = gS[e];
    const float gamma = a.decay[h];
    const float kscale = 1.0f / sqrtf((float)d);
    const int Hd = a.H * d, Hv = a.H * vd;
    for (int t = a.seq_start[s]; t < a.seq_start[s + 1]; ++t) {
        const float* row = a.proj + (size_t)t * a.ld;
        __syncthreads();
        for (int e = threadIdx.x; e < d; e += blockDim.x) {
            qk[e] = row[h * d + e];
            qk[d + e] = row[Hd + h * d + e] * kscale;
        }
        __syncthreads();
        float part = 0.0f;
        if (j < vd) {
            const float v = row[2 * Hd + h * vd + j];
            for (int i = y; i < d; i += DY) {
                const float sv = fmaf(gamma, S[i * vd + j], qk[d + i] * v);
                S[i * vd + j] = sv;
                part = fmaf(sv, qk[i], part);
            }
        }
        red[y * vdr + j] = part;
        __syncthreads();
        if (y == 0) {
            float sum = 0.0f;
            for (int yy = 0; yy < DY; ++yy) sum += red[yy * vdr + j];
            o[j] = j < vd ? sum : 0.0f;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            float ss = 0.0f;
            for (int c = threadIdx.x; c < vd; c += 32) ss = fmaf(o[c], o[c], ss);
            ss = sp_warp_sum(ss);
            if (threadIdx.x == 0) inv_rms = 1.0f / sqrtf(ss / (float)vd + a.eps);
        }
        __syncthreads();
        if (y == 0 && j < vd)
            sp_st_dt(a.out, a.out_dt, (size_t)t * Hv + h * vd + j, o[j] * inv_rms * sm_silu(row[2 * Hd + Hv + h * vd + j]));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < d * vd; e += blockDim.x) gS[e] = S[e];
}

static SpPerDevice retention_ready;

SP_API int sp_retention(const float* proj, int ld, float* state, int n_slots, const float* decay, void* out, int out_dt,
                        const int* seq_start, const int* seq_slot, int B, int H, int d, int vd, float eps,
                        cudaStream_t stream) {
    if (B <= 0) return 0;
    if (d <= 0 || vd <= 0 || vd > 1024) SP_FAIL("retention: sizes d %d, vd %d are outside this kernel's range", d, vd);
    const int vdr = (vd + 31) / 32 * 32;
    int DY = 256 / vdr;
    if (DY < 1) DY = 1;
    if (DY > d) DY = d;
    const size_t smem = ((size_t)d * vd + 2 * d + (size_t)DY * vdr + vdr) * sizeof(float);
    if (smem > 220 * 1024) SP_FAIL("retention: a state of %d x %d does not fit shared memory", d, vd);
    if (!retention_ready.done()) {
        if (cudaFuncSetAttribute(retention_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess)
            SP_FAIL("retention: cannot raise the shared memory limit");
        retention_ready.mark();
    }
    RetArgs a{proj, ld, state, decay, out, out_dt, seq_start, seq_slot, B, H, d, vd, n_slots, eps};
    retention_scan_kernel<<<dim3(B, H), vdr * DY, smem, stream>>>(a, vdr, DY);
    SP_CHECK_LAUNCH("retention");
    return 0;
}

// ============================================================== retention of a prompt step, in chunks of 64 tokens
// The recurrence unrolled over a chunk that starts at token t0 with the state S (all sums in 32-bit FFMA):
//   o_{t0+i} = γ^{i+1} · Sᵀ q_i  +  Σ_{j ≤ i} γ^{i−j} (q_i · k_j) v_j            (k already divided by √d)
//   S'       = γ^{n} · S  +  Σ_j γ^{n−1−j} k_j v_jᵀ                               (n tokens in the chunk)
// Four launches: (A) every chunk's own Σ_j γ^{n−1−j} k_j v_jᵀ, in parallel; (B) per (sequence, head) the chunks'
// start states one after the other (element by element, cheap), the last one becomes the slot's state; (C) every
// chunk's outputs from its start state, in parallel; (D) unit rms per head, the gate, the store. A chunk's arithmetic
// depends on where the chunk starts in its step only, so the same tokens cut into other steps differ by rounding.
// All products are tiles of out[m][n] = Σ_k a[k][m]·b[k][n] with a and b in shared memory, k-major, 16 x 16 threads
// owning 4·MA x 4·NB outputs each.
#define RC_CHUNK 64
#define RC_TS 68               // row stride of the transposed 64-token arrays

template <int MA, int NB>
__device__ __forceinline__ void rc_mm(const float* __restrict__ a, int lda, const float* __restrict__ b, int ldb, int K,
                                      float (&acc)[4 * MA][4 * NB], int ty, int tx) {
    for (int k = 0; k < K; ++k) {
        float4 av[MA], bv[NB];
#pragma unroll
        for (int i = 0; i < MA; ++i) av[i] = *(const float4*)(a + (size_t)k * lda + 4 * ty + 64 * i);
#pragma unroll
        for (int j = 0; j < NB; ++j) bv[j] = *(const float4*)(b + (size_t)k * ldb + 4 * tx + 64 * j);
#pragma unroll
        for (int i = 0; i < MA; ++i) {
            const float am[4] = {av[i].x, av[i].y, av[i].z, av[i].w};
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const float bn[4] = {bv[j].x, bv[j].y, bv[j].z, bv[j].w};
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int v = 0; v < 4; ++v) acc[4 * i + u][4 * j + v] = fmaf(am[u], bn[v], acc[4 * i + u][4 * j + v]);
            }
        }
    }
}

struct RcArgs {
    const float* proj; int ld;         // rows [q | k | v | g]
    float* state;                      // [slots][H][d][vd]
    const float* decay;                // [H]
    float* chunk_state;                // [chunks][H][d][vd]: (A) the chunk's own sum, (B) turns it into its start state
    float* o_raw;                      // [T][H·vd]
    void* out; int out_dt;
    const int* seq_start; const int* seq_slot;
    int B, H, d, vd, n_slots, n_chunks;
    float eps;
};

// which sequence, which chunk of it, its first token and its length
__device__ __forceinline__ bool rc_chunk_of(const RcArgs& a, int x, int& s, int& t0, int& n) {
    for (s = 0; s < a.B; ++s) {
        const int first = a.seq_start[s], cnt = a.seq_start[s + 1] - first;
        const int nc = (cnt + RC_CHUNK - 1) / RC_CHUNK;
        if (x < nc) {
            t0 = first + x * RC_CHUNK;
            n = min(RC_CHUNK, cnt - x * RC_CHUNK);
            return true;
        }
        x -= nc;
    }
    return false;
}

// (A) grid (chunks, H, column blocks of 64·NB); MA = ceil(d / 64)
template <int MA, int NB>
__global__ void __launch_bounds__(256) retention_chunk_sum_kernel(RcArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int DP = 64 * MA, NP = 64 * NB;
    float* kd = sm;                    // [64][DP]   γ^{n−1−j} k_j / √d
    float* vv = kd + RC_CHUNK * DP;    // [64][NP]
    __shared__ float pw[RC_CHUNK + 1];
    int s, t0, n;
    if (!rc_chunk_of(a, blockIdx.x, s, t0, n)) return;
    const int h = blockIdx.y, c0 = blockIdx.z * NP;
    const int d = a.d, vd = a.vd, Hd = a.H * d;
    const float gamma = a.decay[h], kscale = 1.0f / sqrtf((float)d);
    if (threadIdx.x <= RC_CHUNK) pw[threadIdx.x] = powf(gamma, (float)threadIdx.x);
    __syncthreads();
    for (int e = threadIdx.x; e < RC_CHUNK * DP; e += 256) {
        const int j = e / DP, i = e - j * DP;
        kd[e] = (j < n && i < d) ? a.proj[(size_t)(t0 + j) * a.ld + Hd + h * d + i] * kscale * pw[n - 1 - j] : 0.0f;
    }
    for (int e = threadIdx.x; e < RC_CHUNK * NP; e += 256) {
        const int j = e / NP, c = e - j * NP;
        vv[e] = (j < n && c0 + c < vd) ? a.proj[(size_t)(t0 + j) * a.ld + 2 * Hd + h * vd + c0 + c] : 0.0f;
    }
    __syncthreads();
    float acc[4 * MA][4 * NB];
#pragma unroll
    for (int i = 0; i < 4 * MA; ++i)
#pragma unroll
        for (int j = 0; j < 4 * NB; ++j) acc[i][j] = 0.0f;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    rc_mm<MA, NB>(kd, DP, vv, NP, n, acc, ty, tx);
    float* dst = a.chunk_state + ((size_t)blockIdx.x * a.H + h) * d * vd;
#pragma unroll
    for (int i = 0; i < 4 * MA; ++i) {
        const int r = 4 * ty + 64 * (i >> 2) + (i & 3);
#pragma unroll
        for (int j = 0; j < 4 * NB; ++j) {
            const int c = c0 + 4 * tx + 64 * (j >> 2) + (j & 3);
            if (r < d && c < vd) dst[(size_t)r * vd + c] = acc[i][j];
        }
    }
}

// (B) grid (B, H, pieces of d·vd): VEC elements per thread, the loads of four chunks in flight at a time
template <int VEC>
__global__ void retention_chunk_scan_kernel(RcArgs a) {
    const int s = blockIdx.x, h = blockIdx.y;
    const int slot = a.seq_slot[s];
    if (slot < 0 || slot >= a.n_slots) return;
    const int e = (blockIdx.z * blockDim.x + threadIdx.x) * VEC;
    if (e >= a.d * a.vd) return;
    int c = 0;                                              // the sequence's first chunk among all chunks of the step
    for (int b = 0; b < s; ++b) c += (a.seq_start[b + 1] - a.seq_start[b] + RC_CHUNK - 1) / RC_CHUNK;
    const int cnt = a.seq_start[s + 1] - a.seq_start[s];
    const int n_chunks = (cnt + RC_CHUNK - 1) / RC_CHUNK;
    const float gamma = a.decay[h];
    const float g_full = powf(gamma, (float)RC_CHUNK), g_last = powf(gamma, (float)(cnt - (n_chunks - 1) * RC_CHUNK));
    const size_t stride = (size_t)a.H * a.d * a.vd;
    float* gS = a.state + ((size_t)slot * a.H + h) * a.d * a.vd + e;
    float* p = a.chunk_state + ((size_t)c * a.H + h) * a.d * a.vd + e;
    float S[VEC];
    if (VEC == 4) { const float4 v = *(const float4*)gS; S[0] = v.x; S[1] = v.y; S[2] = v.z; S[3] = v.w; }
    else S[0] = *gS;
    for (int x0 = 0; x0 < n_chunks; x0 += 4) {
        float own[4][VEC];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (x0 + u >= n_chunks) break;
            if (VEC == 4) {
                const float4 v = *(const float4*)(p + (size_t)(x0 + u) * stride);
                own[u][0] = v.x; own[u][1] = v.y; own[u][2] = v.z; own[u][3] = v.w;
            } else own[u][0] = p[(size_t)(x0 + u) * stride];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (x0 + u >= n_chunks) break;
            if (VEC == 4) *(float4*)(p + (size_t)(x0 + u) * stride) = make_float4(S[0], S[1], S[2], S[3]);
            else p[(size_t)(x0 + u) * stride] = S[0];
            const float gn = x0 + u == n_chunks - 1 ? g_last : g_full;
#pragma unroll
            for (int i = 0; i < VEC; ++i) S[i] = fmaf(gn, S[i], own[u][i]);
        }
    }
    if (VEC == 4) *(float4*)gS = make_float4(S[0], S[1], S[2], S[3]);
    else *gS = S[0];
}

// (C) grid (chunks, H, column blocks of 64·NB); MA = ceil(d / 64) sizes the shared arrays only
template <int NB>
__global__ void __launch_bounds__(256) retention_chunk_out_kernel(RcArgs a, int DP) {
    extern __shared__ __align__(16) float sm[];
    const int NP = 64 * NB;
    float* qT = sm;                         // [DP][RC_TS]  (rows padded: the transposed stores then spread over the banks)
    float* kT = qT + (size_t)DP * RC_TS;    // [DP][RC_TS]  k / √d
    float* S = kT + (size_t)DP * RC_TS;     // [DP][NP]
    float* vv = S + (size_t)DP * NP;        // [64][NP]
    float* pT = vv + 64 * NP;               // [64 keys][64 queries]
    __shared__ float pw[RC_CHUNK + 1];
    int s, t0, n;
    if (!rc_chunk_of(a, blockIdx.x, s, t0, n)) return;
    const int h = blockIdx.y, c0 = blockIdx.z * NP;
    const int d = a.d, vd = a.vd, Hd = a.H * d;
    const float gamma = a.decay[h], kscale = 1.0f / sqrtf((float)d);
    if (threadIdx.x <= RC_CHUNK) pw[threadIdx.x] = powf(gamma, (float)threadIdx.x);
    for (int e = threadIdx.x; e < RC_CHUNK * DP; e += 256) {
        const int j = e / DP, i = e - j * DP;               // token j, dim i: read along the dims, store transposed
        const bool ok = j < n && i < d;
        const float* row = a.proj + (size_t)(t0 + j) * a.ld;
        qT[i * RC_TS + j] = ok ? row[h * d + i] : 0.0f;
        kT[i * RC_TS + j] = ok ? row[Hd + h * d + i] * kscale : 0.0f;
    }
    const float* gS = a.chunk_state + ((size_t)blockIdx.x * a.H + h) * d * vd;
    for (int e = threadIdx.x; e < DP * NP; e += 256) {
        const int i = e / NP, c = e - i * NP;
        S[e] = (i < d && c0 + c < vd) ? gS[(size_t)i * vd + c0 + c] : 0.0f;
    }
    for (int e = threadIdx.x; e < RC_CHUNK * NP; e += 256) {
        const int j = e / NP, c = e - j * NP;
        vv[e] = (j < n && c0 + c < vd) ? a.proj[(size_t)(t0 + j) * a.ld + 2 * Hd + h * vd + c0 + c] : 0.0f;
    }
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    {
        // pT[j][i] = γ^{i−j} q_i · k_j for j ≤ i (keys as the rows of the product, so that a thread stores whole float4)
        float p[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int v = 0; v < 4; ++v) p[u][v] = 0.0f;
        rc_mm<1, 1>(kT, RC_TS, qT, RC_TS, d, p, ty, tx);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = 4 * ty + u;
            float r[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const int i = 4 * tx + v;
                r[v] = (j <= i && i < n) ? p[u][v] * pw[i - j] : 0.0f;
            }
            *(float4*)(pT + j * 64 + 4 * tx) = make_float4(r[0], r[1], r[2], r[3]);
        }
    }
    __syncthreads();
    float inter[4][4 * NB], intra[4][4 * NB];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4 * NB; ++v) inter[u][v] = intra[u][v] = 0.0f;
    rc_mm<1, NB>(qT, RC_TS, S, NP, d, inter, ty, tx);
    rc_mm<1, NB>(pT, 64, vv, NP, n, intra, ty, tx);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = 4 * ty + u;
        if (i >= n) continue;
        const float gi = pw[i + 1];
#pragma unroll
        for (int v = 0; v < 4 * NB; ++v) {
            const int c = c0 + 4 * tx + 64 * (v >> 2) + (v & 3);
            if (c < vd) a.o_raw[(size_t)(t0 + i) * a.H * vd + h * vd + c] = fmaf(gi, inter[u][v], intra[u][v]);
        }
    }
}

// (D) grid (T, H): unit rms over the head's values, the gate, the store
__global__ void retention_finish_kernel(RcArgs a, int T) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, h = blockIdx.y;
    const int vd = a.vd, Hv = a.H * vd;
    const float* o = a.o_raw + (size_t)t * Hv + h * vd;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < vd; c += blockDim.x) ss = fmaf(o[c], o[c], ss);
    ss = sp_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)vd + a.eps);
    const float* g = a.proj + (size_t)t * a.ld + 2 * a.H * a.d + Hv + h * vd;
    for (int c = threadIdx.x; c < vd; c += blockDim.x)
        sp_st_dt(a.out, a.out_dt, (size_t)t * Hv + h * vd + c, o[c] * inv * sm_silu(g[c]));
}

SP_API int sp_retention_chunked_supported(int d, int vd) { return d > 0 && d <= 128 && vd > 0; }

SP_API long long sp_retention_chunked_scratch_floats(int n_chunks, int T, int H, int d, int vd) {
    return (long long)n_chunks * H * d * vd + (long long)T * H * vd;
}

SP_API int sp_retention_chunked(const float* proj, int ld, float* state, int n_slots, const float* decay, float* scratch,
                                void* out, int out_dt, const int* seq_start, const int* seq_slot, int B, int T, int n_chunks,
                                int H, int d, int vd, float eps, cudaStream_t stream) {
    if (B <= 0 || T <= 0 || n_chunks <= 0) return 0;
    if (!sp_retention_chunked_supported(d, vd)) SP_FAIL("retention (chunks): key size %d is beyond this kernel's limit 128", d);
    RcArgs a{proj, ld, state, decay, scratch, scratch + (size_t)n_chunks * H * d * vd, out, out_dt, seq_start, seq_slot,
             B, H, d, vd, n_slots, n_chunks, eps};
    const int MA = d <= 64 ? 1 : 2, NB = vd <= 64 ? 1 : 2;
    const int DP = 64 * MA, NP = 64 * NB;
    const dim3 grid(n_chunks, H, (vd + NP - 1) / NP);
    const size_t smem_a = (size_t)(RC_CHUNK * DP + RC_CHUNK * NP) * sizeof(float);
    const size_t smem_c = ((size_t)2 * DP * RC_TS + (size_t)DP * NP + 64 * NP + 64 * 64) * sizeof(float);
    static SpPerDevice ready;
    if (!ready.done()) {
        const int big = 200 * 1024;
        if (cudaFuncSetAttribute(retention_chunk_sum_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, big) != cudaSuccess ||
            cudaFuncSetAttribute(retention_chunk_sum_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, big) != cudaSuccess ||
            cudaFuncSetAttribute(retention_chunk_sum_kernel<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, big) != cudaSuccess ||
            cudaFuncSetAttribute(retention_chunk_sum_kernel<2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, big) != cudaSuccess ||
            cudaFuncSetAttribute(retention_chunk_out_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, big) != cudaSuccess ||
            cudaFuncSetAttribute(retention_chunk_out_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, big) != cudaSuccess)
            SP_FAIL("retention (chunks): cannot raise the shared memory limit");
        ready.mark();
    }
    if (MA == 1 && NB == 1) retention_chunk_sum_kernel<1, 1><<<grid, 256, smem_a, stream>>>(a);
    else if (MA == 1) retention_chunk_sum_kernel<1, 2><<<grid, 256, smem_a, stream>>>(a);
    else if (NB == 1) retention_chunk_sum_kernel<2, 1><<<grid, 256, smem_a, stream>>>(a);
    else retention_chunk_sum_kernel<2, 2><<<grid, 256, smem_a, stream>>>(a);
    SP_CHECK_LAUNCH("retention_chunk_sum");
    if (vd % 4 == 0 && (((uintptr_t)state | (uintptr_t)scratch) & 15) == 0)
        retention_chunk_scan_kernel<4><<<dim3(B, H, (d * vd / 4 + 127) / 128), 128, 0, stream>>>(a);
    else
        retention_chunk_scan_kernel<1><<<dim3(B, H, (d * vd + 255) / 256), 256, 0, stream>>>(a);
    SP_CHECK_LAUNCH("retention_chunk_scan");
    if (NB == 1) retention_chunk_out_kernel<1><<<grid, 256, smem_c, stream>>>(a, DP);
    else retention_chunk_out_kernel<2><<<grid, 256, smem_c, stream>>>(a, DP);
    SP_CHECK_LAUNCH("retention_chunk_out");
    retention_finish_kernel<<<dim3(T, H), 128, 0, stream>>>(a, T);
    SP_CHECK_LAUNCH("retention_finish");
    return 0;
}

// ============================================================== retention of a decode step (one token per sequence)
// The state is streamed once: grid (sequences, heads, blocks of 32 value columns), thread (j, y) takes column j of
// the rows i ≡ y (mod 8) straight from and to global memory; the eight partial sums of a column are added in the
// order of y. The unit rms over all of a head's columns and the gate follow in ``retention_finish_kernel``.
__global__ void __launch_bounds__(256) retention_step_kernel(RcArgs a) {
    extern __shared__ float sm[];
    float* qk = sm;                        // q [d], k/√d [d]
    float* red = qk + 2 * a.d;             // [8][32]
    const int s = blockIdx.x, h = blockIdx.y;
    const int slot = a.seq_slot[s];
    if (slot < 0 || slot >= a.n_slots) return;
    const int t = a.seq_start[s];
    const int d = a.d, vd = a.vd, Hd = a.H * d;
    const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
    const int j = blockIdx.z * 32 + x;
    const float* row = a.proj + (size_t)t * a.ld;
    const float kscale = 1.0f / sqrtf((float)d), gamma = a.decay[h];
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        qk[e] = row[h * d + e];
        qk[d + e] = row[Hd + h * d + e] * kscale;
    }
    __syncthreads();
    float part = 0.0f;
    if (j < vd) {
        const float v = row[2 * Hd + h * vd + j];
        float* gS = a.state + ((size_t)slot * a.H + h) * d * vd + j;
        for (int i0 = y; i0 < d; i0 += 32) {
            float st[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) st[u] = i0 + 8 * u < d ? gS[(size_t)(i0 + 8 * u) * vd] : 0.0f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + 8 * u;
                if (i >= d) break;
                const float sv = fmaf(gamma, st[u], qk[d + i] * v);
                gS[(size_t)i * vd] = sv;
                part = fmaf(sv, qk[i], part);
            }
        }
    }
    red[y * 32 + x] = part;
    __syncthreads();
    if (y == 0 && j < vd) {
        float sum = 0.0f;
#pragma unroll
        for (int yy = 0; yy < 8; ++yy) sum += red[yy * 32 + x];
        a.o_raw[(size_t)t * a.H * vd + h * vd + j] = sum;
    }
}

SP_API int sp_retention_step(const float* proj, int ld, float* state, int n_slots, const float* decay, float* o_raw,
                             void* out, int out_dt, const int* seq_start, const int* seq_slot, int B, int H, int d, int vd,
                             float eps, cudaStream_t stream) {
    if (B <= 0) return 0;
    RcArgs a{proj, ld, state, decay, nullptr, o_raw, out, out_dt, seq_start, seq_slot, B, H, d, vd, n_slots, 0, eps};
    const size_t smem = ((size_t)2 * d + 256) * sizeof(float);
    if (smem > 48 * 1024) SP_FAIL("retention (step): key size %d is beyond this kernel's range", d);
    retention_step_kernel<<<dim3(B, H, (vd + 31) / 32), 256, smem, stream>>>(a);
    SP_CHECK_LAUNCH("retention_step");
    retention_finish_kernel<<<dim3(B, H), 128, 0, stream>>>(a, B);
    SP_CHECK_LAUNCH("retention_finish");
    return 0;
}

// ============================================================== minGRU, token by token
// proj row (32-bit) = [z: W | x: W | g: W] without the biases. One thread per (sequence, channel).
__global__ void mingru_scan_kernel(const float* __restrict__ proj, const void* __restrict__ zb, const void* __restrict__ xb,
                                   int b_dt, float* __restrict__ state, int n_slots, void* __restrict__ out, int out_dt,
                                   const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int B, int W) {
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= B || c >= W) return;
    const int slot = seq_slot[s];
    if (slot < 0 || slot >= n_slots) return;
    const float bz = sp_ld_dt(zb, b_dt, c), bx = sp_ld_dt(xb, b_dt, c);
    float S = state[(size_t)slot * W + c];
    for (int t = seq_start[s]; t < seq_start[s + 1]; ++t) {
        const float* row = proj + (size_t)t * 3 * W;
        const float z = sm_sigmoid(row[c] + bz);
        const float u = row[W + c] + bx;
        const float cand = u >= 0.0f ? u + 0.5f : sm_sigmoid(u);
        S = (1.0f - z) * S + z * cand;
        sp_st_dt(out, out_dt, (size_t)t * W + c, S * sm_silu(row[2 * W + c]));
    }
    state[(size_t)slot * W + c] = S;
}

SP_API int sp_mingru(const float* proj, const void* zb, const void* xb, int b_dt, float* state, int n_slots, void* out,
                     int out_dt, const int* seq_start, const int* seq_slot, int B, int W, cudaStream_t stream) {
    if (B <= 0) return 0;
    const int threads = 128;
    mingru_scan_kernel<<<dim3((W + threads - 1) / threads, B), threads, 0, stream>>>(proj, zb, xb, b_dt, state, n_slots, out,
                                                                                    out_dt, seq_start, seq_slot, B, W);
    SP_CHECK_LAUNCH("mingru");
    return 0;
}

// ============================================================== minGRU of a prompt step, in chunks of 32 tokens
// S_t = a_t S_{t-1} + b_t with a_t = 1 − z_t, b_t = z_t c_t composes: over a chunk S_end = A·S_start + Bsum with
// A = Π a_t and Bsum the chunk run from zero. (1) every (chunk, channel) finds (A, Bsum); (2) per (sequence, channel)
// the chunks' start states one after the other; (3) every (chunk, channel) runs again from its start state and writes.
#define MG_CHUNK 32

__device__ __forceinline__ bool mg_chunk_of(const int* seq_start, int B, int x, int& s, int& t0, int& n) {
    for (s = 0; s < B; ++s) {
        const int first = seq_start[s], cnt = seq_start[s + 1] - first;
        const int nc = (cnt + MG_CHUNK - 1) / MG_CHUNK;
        if (x < nc) {
            t0 = first + x * MG_CHUNK;
            n = min(MG_CHUNK, cnt - x * MG_CHUNK);
            return true;
        }
        x -= nc;
    }
    return false;
}

// PASS 1: scratch[chunk][c] = (A, Bsum).  PASS 3: reads scratch[chunk][c].x as the start state and writes the outputs.
template <int PASS>
__global__ void mingru_chunk_kernel(const float* __restrict__ proj, const void* __restrict__ zb, const void* __restrict__ xb,
                                    int b_dt, float2* __restrict__ scratch, void* __restrict__ out, int out_dt,
                                    const int* __restrict__ seq_start, int B, int W) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    int s, t0, n;
    if (c >= W || !mg_chunk_of(seq_start, B, blockIdx.y, s, t0, n)) return;
    const float bz = sp_ld_dt(zb, b_dt, c), bx = sp_ld_dt(xb, b_dt, c);
    float2* cell = scratch + (size_t)blockIdx.y * W + c;
    float S = PASS == 1 ? 0.0f : cell->x, A = 1.0f;
    for (int tb = t0; tb < t0 + n; tb += 8) {
        float pz[8], px[8], pg[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {                        // eight tokens' loads in flight
            const bool in = tb + i < t0 + n;
            const float* row = proj + (size_t)(in ? tb + i : tb) * 3 * W;
            pz[i] = row[c];
            px[i] = row[W + c];
            pg[i] = PASS == 1 ? 0.0f : row[2 * W + c];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (tb + i >= t0 + n) break;
            const float z = sm_sigmoid(pz[i] + bz);
            const float u = px[i] + bx;
            const float cand = u >= 0.0f ? u + 0.5f : sm_sigmoid(u);
            S = (1.0f - z) * S + z * cand;
            if (PASS == 1) A *= 1.0f - z;
            else sp_st_dt(out, out_dt, (size_t)(tb + i) * W + c, S * sm_silu(pg[i]));
        }
    }
    if (PASS == 1) *cell = make_float2(A, S);
}

__global__ void mingru_chunk_scan_kernel(float2* __restrict__ scratch, float* __restrict__ state, int n_slots,
                                         const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int B, int W) {
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= B || c >= W) return;
    const int slot = seq_slot[s];
    if (slot < 0 || slot >= n_slots) return;
    int chunk = 0;
    for (int b = 0; b < s; ++b) chunk += (seq_start[b + 1] - seq_start[b] + MG_CHUNK - 1) / MG_CHUNK;
    const int cnt = seq_start[s + 1] - seq_start[s];
    float S = state[(size_t)slot * W + c];
    const int n_chunks = (cnt + MG_CHUNK - 1) / MG_CHUNK;
    for (int x0 = 0; x0 < n_chunks; x0 += 8) {
        float2 ab[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (x0 + u < n_chunks) ab[u] = scratch[(size_t)(chunk + x0 + u) * W + c];      // eight cells in flight
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (x0 + u >= n_chunks) break;
            scratch[(size_t)(chunk + x0 + u) * W + c].x = S;
            S = fmaf(ab[u].x, S, ab[u].y);
        }
    }
    state[(size_t)slot * W + c] = S;
}

SP_API int sp_mingru_chunk_tokens() { return MG_CHUNK; }

SP_API int sp_mingru_chunked(const float* proj, const void* zb, const void* xb, int b_dt, float* state, int n_slots,
                             float* scratch, void* out, int out_dt, const int* seq_start, const int* seq_slot, int B,
                             int n_chunks, int W, cudaStream_t stream) {
    if (B <= 0 || n_chunks <= 0) return 0;
    const int threads = 128;
    const dim3 grid((W + threads - 1) / threads, n_chunks);
    mingru_chunk_kernel<1><<<grid, threads, 0, stream>>>(proj, zb, xb, b_dt, (float2*)scratch, out, out_dt, seq_start, B, W);
    SP_CHECK_LAUNCH("mingru_chunk_1");
    mingru_chunk_scan_kernel<<<dim3((W + threads - 1) / threads, B), threads, 0, stream>>>((float2*)scratch, state, n_slots,
                                                                                         seq_start, seq_slot, B, W);
    SP_CHECK_LAUNCH("mingru_chunk_scan");
    mingru_chunk_kernel<3><<<grid, threads, 0, stream>>>(proj, zb, xb, b_dt, (float2*)scratch, out, out_dt, seq_start, B, W);
    SP_CHECK_LAUNCH("mingru_chunk_3");
    return 0;
}

// ============================================================== PolyNorm
// out = a·z/rms(z) + b·z²/rms(z²) + c·z³/rms(z³) + e over each row of z (32-bit), rms with eps inside the root.
__global__ void __launch_bounds__(256)
polynorm_kernel(const float* __restrict__ z, const void* __restrict__ coef, int c_dt, void* __restrict__ out, int out_dt,
                int T, int F, float eps) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    if (t >= T) return;
    const float* row = z + (size_t)t * F;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    const bool vec = (F & 3) == 0 && (((uintptr_t)z) & 15) == 0;
    if (vec) {
        for (int c = threadIdx.x * 4; c < F; c += blockDim.x * 4) {
            const float4 q = *(const float4*)(row + c);
            const float e[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float v = e[i], v2 = v * v, v3 = v2 * v;
                s2 = fmaf(v, v, s2);
                s4 = fmaf(v2, v2, s4);
                s6 = fmaf(v3, v3, s6);
            }
        }
    } else
    for (int c = threadIdx.x; c < F; c += blockDim.x) {
        const float v = row[c], v2 = v * v, v3 = v2 * v;
        s2 = fmaf(v, v, s2);
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v3, v3, s6);
    }
    s2 = sp_block_sum(s2, scratch);
    s4 = sp_block_sum(s4, scratch);
    s6 = sp_block_sum(s6, scratch);
    const float r1 = 1.0f / sqrtf(s2 / (float)F + eps), r2 = 1.0f / sqrtf(s4 / (float)F + eps), r3 = 1.0f / sqrtf(s6 / (float)F + eps);
    const float ca = sp_ld_dt(coef, c_dt, 0), cb = sp_ld_dt(coef, c_dt, 1), cc = sp_ld_dt(coef, c_dt, 2), ce = sp_ld_dt(coef, c_dt, 3);
    if (vec) {
        for (int c = threadIdx.x * 4; c < F; c += blockDim.x * 4) {
            const float4 q = *(const float4*)(row + c);
            const float e[4] = {q.x, q.y, q.z, q.w};
            float o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float v = e[i], v2 = v * v, v3 = v2 * v;
                o[i] = ca * (v * r1) + cb * (v2 * r2) + cc * (v3 * r3) + ce;
            }
            if (out_dt == SP_DT_F32) *(float4*)((float*)out + (size_t)t * F + c) = make_float4(o[0], o[1], o[2], o[3]);
            else {
                __nv_bfloat162 p0 = __floats2bfloat162_rn(o[0], o[1]), p1 = __floats2bfloat162_rn(o[2], o[3]);
                uint2 pk;
                pk.x = *(uint32_t*)&p0; pk.y = *(uint32_t*)&p1;
                *(uint2*)((__nv_bfloat16*)out + (size_t)t * F + c) = pk;
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < F; c += blockDim.x) {
        const float v = row[c], v2 = v * v, v3 = v2 * v;
        sp_st_dt(out, out_dt, (size_t)t * F + c, ca * (v * r1) + cb * (v2 * r2) + cc * (v3 * r3) + ce);
    }
}

SP_API int sp_polynorm(const float* z, const void* coef, int c_dt, void* out, int out_dt, int T, int F, float eps,
                       cudaStream_t stream) {
    if (T <= 0) return 0;
    polynorm_kernel<<<T, 256, 0, stream>>>(z, coef, c_dt, out, out_dt, T, F, eps);
    SP_CHECK_LAUNCH("polynorm");
    return 0;
}

// ============================================================== rows += bias
__global__ void add_bias_kernel(float* __restrict__ x, const void* __restrict__ bias, int b_dt, size_t n, int N) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += sp_ld_dt(bias, b_dt, i % N);
}

SP_API int sp_add_bias(float* x, const void* bias, int b_dt, int T, int N, cudaStream_t stream) {
    const size_t n = (size_t)T * N;
    if (n == 0) return 0;
    add_bias_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, bias, b_dt, n, N);
    SP_CHECK_LAUNCH("add_bias");
    return 0;
}
