// Differential attention of a prompt step on the tensor cores (mma.sync m16n8k16, bfloat16 in, 32-bit accumulation).
//
// One CTA of four warps takes 64 queries of one sequence and one head, BOTH maps: the query tile [64][2·D] and, page by
// page, the key tile [64][2·D] and the value tile [64][VD] of the head's kv head (cp.async, two stages). For each
// map the warp computes S = Q_m · K_mᵀ for its 16 rows, scales, caps (c·tanh(s/c)), masks and runs the online softmax
// in 32-bit; P (rounded to bfloat16 like every operand of a tensor-core product here) times V is added to the map's
// own accumulator, so a value tile is fetched once for both maps. At the end o = a1 − λ·a2 is brought to unit rms
// over the head's VD values and scaled by a constant.
//
// Visibility: a query at position p sees key j ≤ p when p − j < window (window 0: always) or j < keep_first. The
// pages walked are those of the kept first keys that lie before the window's first page, then the window's own.
#include "flash_common.cuh"

SP_API const char* sp_diff_flash_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(diff_flash)

namespace {

struct DiffKV {
    const __nv_bfloat16* k;     // [pages][G][64][2·D]
    const __nv_bfloat16* v;     // [pages][G][64][VD]
    const int* page_table;      // [rows][max_pages]
    const int* seq_row;         // [B]
    int max_pages;
    int G;
    SpRange rg;
};

struct DiffConst {
    int H, window, keep_first;
    float scale, softcap, lam, eps, out_scale;
};

// tanh by one exponential: 1 − 2 / (1 + e^{2x}); exact at ±inf, absolute error of a few 1e-7
__device__ __forceinline__ float tanh_by_exp(float x) {
    return 1.0f - __fdividef(2.0f, 1.0f + fast_exp2(x * (2.0f * LOG2E)));
}

// One map of one warp's 16 query rows against the 64 keys of a tile. ``m`` is the running maximum in the log2 domain.
template <int D, int VD, bool MASKED>
__device__ __forceinline__ void diff_step(uint32_t q_tile, int q_row0, int map, uint32_t k_tile, uint32_t v_tile,
                                          int tile_pos0, const int (&lo)[2], const int (&hi)[2], const DiffConst& c,
                                          float (&o)[VD / 8][4], float (&m)[2], float (&l)[2], int lane) {
    using TK = Tile<2 * D>;
    using TV = Tile<VD>;
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        {
            const int row = q_row0 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int d = map * D + kk * 16 + ((lane >> 4) << 3);
            ldmatrix_x4(q_tile + row * TK::ROW + d * 2, a[0], a[1], a[2], a[3]);
        }
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            const int key = np * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int d = map * D + kk * 16 + (((lane >> 3) & 1) << 3);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_tile + key * TK::ROW + d * 2, b0, b1, b2, b3);
            mma_bf16(s[2 * np], a, b0, b1);
            mma_bf16(s[2 * np + 1], a, b2, b3);
        }
    }
    const int t = lane & 3;
    const float inv_cap = c.softcap > 0.0f ? 1.0f / c.softcap : 0.0f;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            float v = s[nt][e] * c.scale;
            if (c.softcap > 0.0f) v = c.softcap * tanh_by_exp(v * inv_cap);
            v *= LOG2E;
            if (MASKED) {
                const int key = tile_pos0 + nt * 8 + 2 * t + (e & 1);
                if (key > hi[r] || (key < lo[r] && key >= c.keep_first)) v = -INFINITY;
            }
            s[nt][e] = v;
            mx[r] = fmaxf(mx[r], v);
        }
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float mnew = fmaxf(m[r], mx[r]);
        msafe[r] = (mnew == -INFINITY) ? 0.0f : mnew;
        corr[r] = fast_exp2(m[r] - msafe[r]);         // m = -inf gives 0
        m[r] = mnew;
    }
    float sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float p = fast_exp2(s[nt][e] - msafe[e >> 1]);
            s[nt][e] = p;
            sum[e >> 1] += p;
        }
    }
    l[0] = l[0] * corr[0] + sum[0];                   // per-lane partial; the four lanes of a row are added at the end
    l[1] = l[1] * corr[1] + sum[1];
#pragma unroll
    for (int i = 0; i < VD / 8; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0];
        o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < VD / 16; ++dp) {
            const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int d = dp * 16 + ((lane >> 4) << 3);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(v_tile + key * TV::ROW + d * 2, b0, b1, b2, b3);
            mma_bf16(o[2 * dp], a, b0, b1);
            mma_bf16(o[2 * dp + 1], a, b2, b3);
        }
    }
}

template <int D, int VD>
constexpr int diff_smem() { return 3 * Tile<2 * D>::BYTES + 2 * Tile<VD>::BYTES; }

template <int D, int VD>
__global__ void __launch_bounds__(128)
diff_flash_prefill_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, DiffKV kv,
                          const int* __restrict__ seq_start, const int* __restrict__ positions, int n_seqs, DiffConst c) {
    using TK = Tile<2 * D>;
    using TV = Tile<VD>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t q_tile = smem_u32(smem);
    const uint32_t k_tiles = q_tile + TK::BYTES;
    const uint32_t v_tiles = k_tiles + 2 * TK::BYTES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    sp_allow_dependents();
    sp_wait_for_predecessor();

    // which sequence and which 64-token tile of it; the tiles with the most keys start first
    int x = (int)gridDim.y - 1 - (int)blockIdx.y, b = 0, first = 0, n_new = 0;
    for (; b < n_seqs; ++b) {
        first = seq_start[b];
        n_new = seq_start[b + 1] - first;
        const int nt = (n_new + KT - 1) / KT;
        if (x < nt) break;
        x -= nt;
    }
    if (b >= n_seqs) return;
    const int t0 = first + x * KT;
    const int n_rows = min(KT, n_new - x * KT);
    const int pos0 = positions[t0];
    const int h = blockIdx.x;
    const int g = h / (c.H / kv.G);
    const int* pt = kv.page_table + (size_t)sp_checked_row(kv.seq_row[b], kv.rg) * kv.max_pages;

    const int last_pos = pos0 + n_rows - 1;
    const int first_key = (c.window > 0 && pos0 - c.window + 1 > 0) ? pos0 - c.window + 1 : 0;
    const int j_lo = first_key / KT, j_hi = last_pos / KT;
    const int kept_pages = min((c.keep_first + KT - 1) / KT, j_lo);       // pages of kept keys in front of the window's
    const int n_tiles = kept_pages + (j_hi - j_lo + 1);
    auto page_of = [&](int i) { return i < kept_pages ? i : j_lo + (i - kept_pages); };
    auto fetch = [&](int i, int stage) {
        const size_t pg = (size_t)sp_checked_page(pt[sp_checked_entry(page_of(i), kv.max_pages, kv.rg)], kv.rg) * kv.G + g;
        load_tile_async<2 * D>(k_tiles + stage * TK::BYTES, kv.k + pg * KT * (2 * D), 2 * D, KT, tid, 128);
        load_tile_async<VD>(v_tiles + stage * TV::BYTES, kv.v + pg * KT * VD, VD, KT, tid, 128);
    };

    load_tile_async<2 * D>(q_tile, q + ((size_t)t0 * c.H + h) * (2 * D), (size_t)c.H * 2 * D, n_rows, tid, 128);
    fetch(0, 0);
    cp_async_commit();

    float o1[VD / 8][4], o2[VD / 8][4];
#pragma unroll
    for (int i = 0; i < VD / 8; ++i) {
        o1[i][0] = o1[i][1] = o1[i][2] = o1[i][3] = 0.0f;
        o2[i][0] = o2[i][1] = o2[i][2] = o2[i][3] = 0.0f;
    }
    float m1[2] = {-INFINITY, -INFINITY}, l1[2] = {0.0f, 0.0f}, m2[2] = {-INFINITY, -INFINITY}, l2[2] = {0.0f, 0.0f};
    const int r0 = warp * 16 + (lane >> 2);
    const int hi[2] = {pos0 + r0, pos0 + r0 + 8};
    const int lo[2] = {c.window > 0 ? hi[0] - c.window + 1 : 0, c.window > 0 ? hi[1] - c.window + 1 : 0};
    const int warp_hi = pos0 + warp * 16 + 15;                     // last key any row of this warp may see
    const int warp_lo = c.window > 0 ? pos0 + warp * 16 - c.window + 1 : 0;
    const bool warp_active = warp * 16 < n_rows;

    for (int i = 0; i < n_tiles; ++i) {
        const int stage = i & 1;
        if (i + 1 < n_tiles) fetch(i + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int tile_pos0 = page_of(i) * KT;
        if (warp_active && tile_pos0 <= warp_hi && (tile_pos0 + KT - 1 >= warp_lo || tile_pos0 < c.keep_first)) {
            // every key of the tile is at or before the warp's first row and inside its last row's window
            const bool all_seen = tile_pos0 + KT - 1 <= pos0 + warp * 16 && (c.window <= 0 || tile_pos0 >= warp_hi - c.window + 1);
            const uint32_t kt = k_tiles + stage * TK::BYTES, vt = v_tiles + stage * TV::BYTES;
            if (all_seen) {
                diff_step<D, VD, false>(q_tile, warp * 16, 0, kt, vt, tile_pos0, lo, hi, c, o1, m1, l1, lane);
                diff_step<D, VD, false>(q_tile, warp * 16, 1, kt, vt, tile_pos0, lo, hi, c, o2, m2, l2, lane);
            } else {
                diff_step<D, VD, true>(q_tile, warp * 16, 0, kt, vt, tile_pos0, lo, hi, c, o1, m1, l1, lane);
                diff_step<D, VD, true>(q_tile, warp * 16, 1, kt, vt, tile_pos0, lo, hi, c, o2, m2, l2, lane);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l1[r] += __shfl_xor_sync(0xffffffffu, l1[r], 1);
        l1[r] += __shfl_xor_sync(0xffffffffu, l1[r], 2);
        l2[r] += __shfl_xor_sync(0xffffffffu, l2[r], 1);
        l2[r] += __shfl_xor_sync(0xffffffffu, l2[r], 2);
    }
    const int t = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + r * 8;
        const float i1 = 1.0f / l1[r], i2 = c.lam / l2[r];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < VD / 8; ++i) {
            o1[i][2 * r] = o1[i][2 * r] * i1 - o2[i][2 * r] * i2;
            o1[i][2 * r + 1] = o1[i][2 * r + 1] * i1 - o2[i][2 * r + 1] * i2;
            ss = fmaf(o1[i][2 * r], o1[i][2 * r], ss);
            ss = fmaf(o1[i][2 * r + 1], o1[i][2 * r + 1], ss);
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        if (row >= n_rows) continue;
        const float inv = c.out_scale / sqrtf(ss / (float)VD + c.eps);
        __nv_bfloat16* dst = out + ((size_t)(t0 + row) * c.H + h) * VD;
#pragma unroll
        for (int i = 0; i < VD / 8; ++i)
            *(uint32_t*)(dst + i * 8 + 2 * t) = pack_bf16(o1[i][2 * r] * inv, o1[i][2 * r + 1] * inv);
    }
}

template <int D, int VD>
int launch_as(dim3 grid, cudaStream_t stream, const __nv_bfloat16* q, __nv_bfloat16* out, const DiffKV& kv,
              const int* seq_start, const int* positions, int n_seqs, const DiffConst& c) {
    static SpPerDevice ok;            // the opt-in holds for one device: asked for on each device's first launch
    if (!ok.done()) {
        cudaError_t e = cudaFuncSetAttribute(diff_flash_prefill_kernel<D, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             diff_smem<D, VD>());
        if (e != cudaSuccess) SP_FAIL("diff_flash: cannot reserve %d bytes of shared memory: %s", diff_smem<D, VD>(), cudaGetErrorString(e));
        ok.mark();
    }
    sp_launch_dependent(diff_flash_prefill_kernel<D, VD>, grid, dim3(128), (size_t)diff_smem<D, VD>(), stream, q, out, kv,
                        seq_start, positions, n_seqs, c);
    return 0;
}

bool size_built(int v) { return v == 16 || v == 32 || v == 64 || v == 128; }
}  // namespace

SP_API int sp_diff_flash_query_tile() { return KT; }

SP_API int sp_diff_flash_supported(int d, int vd, int H, int G, int page_size) {
    return size_built(d) && size_built(vd) && G > 0 && H % G == 0 && page_size == KT;
}

SP_API int sp_diff_flash_prefill(const void* q, void* out, const void* kpool, const void* vpool, const int* seq_start,
                                 const int* positions, const int* seq_row, const int* page_table, int max_pages,
                                 int page_size, int n_seqs, int n_q_tiles, int H, int G, int d, int vd, int window,
                                 int keep_first, float scale, float softcap, float lam, float eps, float out_scale,
                                 cudaStream_t stream) {
    if (n_q_tiles <= 0) return 0;
    if (!sp_diff_flash_supported(d, vd, H, G, page_size))
        SP_FAIL("diff_flash: sizes d %d, vd %d, heads %d/%d, page %d are not built", d, vd, H, G, page_size);
    DiffKV kv{(const __nv_bfloat16*)kpool, (const __nv_bfloat16*)vpool, page_table, seq_row, max_pages, G, sp_range_host};
    DiffConst c{H, window > 0 ? window : 0, (window > 0 && keep_first > 0) ? keep_first : 0, scale, softcap, lam, eps, out_scale};
    const dim3 grid(H, n_q_tiles);
    const __nv_bfloat16* qq = (const __nv_bfloat16*)q;
    __nv_bfloat16* oo = (__nv_bfloat16*)out;
#define DF_CASE(DD, VV) \
    if (d == DD && vd == VV) { if (launch_as<DD, VV>(grid, stream, qq, oo, kv, seq_start, positions, n_seqs, c)) return 1; } else
#define DF_ROW(DD) DF_CASE(DD, 16) DF_CASE(DD, 32) DF_CASE(DD, 64) DF_CASE(DD, 128)
    DF_ROW(16) DF_ROW(32) DF_ROW(64) DF_ROW(128)
    SP_FAIL("diff_flash: sizes d %d, vd %d are not built", d, vd);
#undef DF_ROW
#undef DF_CASE
    SP_CHECK_LAUNCH("diff_flash_prefill");
    return 0;
}
