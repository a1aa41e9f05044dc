// Differential attention over the paged cache on the tensor cores (bfloat16 in, 32-bit softmax and sums).
//
// Every head has two maps of queries and keys over one set of values: a_m = softmax(scale q_m k_m^T) v for m = 1, 2,
// o = a_1 - lam a_2, out = out_scale * o / sqrt(mean(o^2) + eps).  Position p sees key j <= p with p - j < window, and
// beside a window the keys below keep_first.
//
// The shape is that of the plain tensor-core attention (attention_mma.cu): a tile of rows (token, head of the group)
// of one head of values, keys in blocks of 64 through a two-stage cp.async pipeline, S = Q K^T and O += P V as mma.sync
// m16n8k16 with P rounded to bfloat16, a running maximum and sum for every row.  What differs: two warps share 16 rows,
// one for each map, so a block of values is brought once for both maps (the keys of the two maps are two heads of the
// key pages, [pages, kv_heads * 2, page_size, D]; values [pages, kv_heads, page_size, DV], DV != D allowed); the blocks
// of a tile are those of the kept first keys that the window has passed, then those from the window's first key; and
// at the end the map-2 warps hand their normalised results through shared memory to the map-1 warps, which subtract,
// norm over the head's values and store.  Prompt portions and single tokens run the same kernel (a single token's
// tile holds the heads of its group).
#include "attention_mma.cuh"
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

struct DiffParams {
    const __nv_bfloat16* y;          // [tokens, y_stride]: q at q_col, [heads, 2, D]
    int y_stride, q_col;
    __nv_bfloat16* out;              // [tokens, out_stride]: the result at out_col, [heads, DV]
    int out_stride, out_col;
    float out_scale;
    const __nv_bfloat16* k_cache;
    const __nv_bfloat16* v_cache;
    const int* cu_q;
    const int* q_start;
    const int* block_table;
    int table_stride;
    const int2* tiles;               // (sequence, first token of the tile among the sequence's new tokens); null: a step of
                                     // single tokens, tile = sequence = token
    int n_pages, heads, kv_heads, page_size, window, keep_first;
    float scale_log2;                // scale * log2(e)
    float lam, sub_eps;
    int tokens_per_tile;
    int* status;
};

namespace {

// (Two CTAs an SM, asked for where a warp's accumulators would leave room (keys of up to 64, values of up to 128: 128
// registers with a few spilled), measured on a B200: a prompt's attention 12 % faster, a decode step's 8 % slower; not taken.)
// SPLIT (tiles of at most 16 rows: single tokens): the four slabs of warps do not take 16 rows each but 16 of a block's 64
// keys each, for the same 16 rows; every warp then walks a quarter of the keys, and at the end the slabs' maxima, sums
// and results meet in shared memory and are merged by the first slab's warps.
template <int D, int DV, int WARPS, bool SPLIT>
__global__ void __launch_bounds__(WARPS * 32)
attention_diff_kernel(const DiffParams p) {
    constexpr int LD = D + 8, LDV = DV + 8;   // padded rows: conflict-free fragment loads, 16-byte aligned rows
    constexpr int THREADS = WARPS * 32;
    constexpr int NJ = SPLIT ? 2 : KB / 8;    // tiles of 8 keys of a block whose scores a warp forms
    constexpr int NK = SPLIT ? 1 : KB / 16;   // steps of 16 keys of a block in a warp's product with the values
    static_assert(!SPLIT || WARPS == 8, "four slabs of two warps share a block's four runs of 16 keys");
    // stages of the copy pipeline: a step of single tokens only streams keys and values, so it keeps one more block in flight
    constexpr int ST = SPLIT ? 3 : 2;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [stages][2 maps][KB][LD]
    __nv_bfloat16* vs = ks + (SPLIT ? 3 : 2) * 2 * KB * LD;              // [stages][KB][LDV]

    pdl_launch();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    const int map = warp & 1, rg = warp >> 1;
    const int kvh = blockIdx.y;
    int seq = blockIdx.x, tok0 = 0;
    if (p.tiles) {
        const int2 tile = p.tiles[blockIdx.x];
        seq = tile.x;
        tok0 = tile.y;
    }
    const int q_begin = p.cu_q[seq];
    const int q_len = p.cu_q[seq + 1] - q_begin;
    const int ntok = min(p.tokens_per_tile, q_len - tok0);
    const int group = p.heads / p.kv_heads;
    if (ntok <= 0) {
        // a step of single tokens padded to a captured graph's size: sequence i without a token is padding token i,
        // whose row of the result is cleared so that what follows reads numbers
        if (!p.tiles) {
            __nv_bfloat16* op = p.out + (size_t)blockIdx.x * p.out_stride + p.out_col + (size_t)kvh * group * DV;
            for (int e = threadIdx.x; e < group * DV; e += THREADS) op[e] = __float2bfloat16_rn(0.f);
        }
        return;
    }
    const int rows_valid = ntok * group;
    const int row_base = SPLIT ? 0 : rg * 16;          // the first of this warp's 16 rows in the tile
    const int key_off = SPLIT ? rg * 16 : 0;           // the first of this warp's keys in a block
    const bool slab_live = SPLIT || rg * 16 < rows_valid;
    const int start = p.q_start[seq];
    const int pos_lo = start + tok0, pos_hi = pos_lo + ntok - 1;
    const int keep = p.window > 0 ? p.keep_first : 0;
    const int key_lo = first_visible_key(pos_lo, p.window, 0) / KB * KB;
    const int key_hi = pos_hi + 1;
    // blocks of the kept first keys that lie before the window's first block, then the window's
    const int nsink = (keep > 0 && key_lo > 0) ? min((keep + KB - 1) / KB, key_lo / KB) : 0;
    const int nblk = nsink + (key_hi - key_lo + KB - 1) / KB;

    // the two rows of this thread
    int pos[2], tok[2], head[2], first[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = row_base + gq + 8 * i;
        valid[i] = row < rows_valid;
        const int tk = valid[i] ? row / group : 0;
        tok[i] = q_begin + tok0 + tk;
        pos[i] = pos_lo + tk;
        first[i] = first_visible_key(pos[i], p.window, 0);
        head[i] = kvh * group + (valid[i] ? row % group : 0);
    }

    // Q fragments of this warp's map
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const __nv_bfloat16* qp = p.y + (size_t)tok[i] * p.y_stride + p.q_col + ((size_t)head[i] * 2 + map) * D;
#pragma unroll
        for (int ks_ = 0; ks_ < D / 16; ++ks_) {
            qf[ks_][i] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp + ks_ * 16 + 2 * tq) : 0u;
            qf[ks_][i + 2] = valid[i] ? *reinterpret_cast<const uint32_t*>(qp + ks_ * 16 + 8 + 2 * tq) : 0u;
        }
    }

    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

    const int* table = p.block_table + (size_t)seq * p.table_stride;
    auto first_key_of = [&](int blk) { return blk < nsink ? blk * KB : key_lo + (blk - nsink) * KB; };
    auto load_block = [&](int blk, int stage) {
        const int kb = first_key_of(blk);
        // the block's four runs of 16 keys lie in one page each
        static_assert(KB == 64, "four runs of 16 keys");
        size_t base_k[4], base_v[4];      // rows of the run's first key (map 0) and first value in the pages
        bool okp[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const int key = kb + 16 * h;
            okp[h] = key < key_hi;
            base_k[h] = base_v[h] = 0;
            if (okp[h]) {
                const int page = table[key / p.page_size];
                // a page between the kept first tokens and the window may be gone already; its keys are masked below
                if (page < 0 || page >= p.n_pages) {
                    okp[h] = false;
                } else {
                    const size_t pv = (size_t)page * p.kv_heads + kvh;
                    base_v[h] = pv * p.page_size + key % p.page_size;
                    base_k[h] = pv * 2 * p.page_size + key % p.page_size;
                }
            }
        }
        constexpr int KC = D / 8, VC = DV / 8;          // 16-byte pieces in a row of keys, of values
        for (int c = threadIdx.x; c < 2 * KB * KC; c += THREADS) {
            const int m = c / (KB * KC), r = (c / KC) % KB, piece = c % KC;
            const int h = r >> 4;                       // selected without indexing, so the bases stay in registers
            const size_t bh = h == 0 ? base_k[0] : h == 1 ? base_k[1] : h == 2 ? base_k[2] : base_k[3];
            const bool oh = h == 0 ? okp[0] : h == 1 ? okp[1] : h == 2 ? okp[2] : okp[3];
            const bool ok = oh && (kb + r) < key_hi;
            const size_t off = ok ? (bh + (size_t)m * p.page_size + (r & 15)) * D + piece * 8 : 0;
            cp_async16(ks + (((size_t)stage * 2 + m) * KB + r) * LD + piece * 8, p.k_cache + off, ok);
        }
        for (int c = threadIdx.x; c < KB * VC; c += THREADS) {
            const int r = c / VC, piece = c % VC;
            const int h = r >> 4;
            const size_t bh = h == 0 ? base_v[0] : h == 1 ? base_v[1] : h == 2 ? base_v[2] : base_v[3];
            const bool oh = h == 0 ? okp[0] : h == 1 ? okp[1] : h == 2 ? okp[2] : okp[3];
            const bool ok = oh && (kb + r) < key_hi;
            const size_t off = ok ? (bh + (r & 15)) * DV + piece * 8 : 0;
            cp_async16(vs + ((size_t)stage * KB + r) * LDV + piece * 8, p.v_cache + off, ok);
        }
    };

    // a group of copies for every block, also an empty one past the last block, so that the count of groups in flight
    // says which block has landed
#pragma unroll
    for (int b = 0; b < ST - 1; ++b) {
        if (b < nblk) load_block(b, b);
        cp_async_commit();
    }
    for (int blk = 0; blk < nblk; ++blk) {
        const int stage = blk % ST;
        if (blk + ST - 1 < nblk) load_block(blk + ST - 1, (blk + ST - 1) % ST);
        cp_async_commit();
        cp_async_wait<ST - 1>();
        __syncthreads();
        if (!slab_live) {                                // a slab without rows (a short tile): copies and barriers only
            __syncthreads();
            continue;
        }
        const __nv_bfloat16* kst = ks + ((size_t)stage * 2 + map) * KB * LD;
        const __nv_bfloat16* vst = vs + (size_t)stage * KB * LDV;
        const int kb = first_key_of(blk);

        // S = Q K^T of this warp's map
        float s[NJ][4];
#pragma unroll
        for (int j = 0; j < NJ; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int ks_ = 0; ks_ < D / 16; ++ks_) {
#pragma unroll
            for (int j = 0; j < NJ; j += 2) {
                uint32_t kf[4];
                const int mat = lane >> 3, r = lane & 7;
                ldmatrix_x4(kf, kst + (size_t)(key_off + (j + (mat >> 1)) * 8 + r) * LD + ks_ * 16 + (mat & 1) * 8);
                mma_bf16(s[j], qf[ks_], kf[0], kf[1]);
                mma_bf16(s[j + 1], qf[ks_], kf[2], kf[3]);
            }
        }
        // mask, running maximum and sum (log2 domain)
        float mnew[2] = {mrow[0], mrow[1]};
        // a block of the window all of whose keys every row of the tile sees needs no mask
        const bool open = blk >= nsink && (kb + KB - 1 <= pos_lo) && kb >= first_visible_key(pos_hi, p.window, 0);
        if (open) {
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[j][e] *= p.scale_log2;
                    mnew[e >> 1] = fmaxf(mnew[e >> 1], s[j][e]);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const int key = kb + key_off + j * 8 + 2 * tq + (e & 1);
                    // a kept first key that the window's own blocks also hold is counted there, not here
                    const bool see = valid[i] && key <= pos[i] &&
                                     (blk < nsink ? (key < keep && key < key_lo) : (key >= first[i] || key < keep));
                    s[j][e] = see ? s[j][e] * p.scale_log2 : -INFINITY;
                    mnew[i] = fmaxf(mnew[i], s[j][e]);
                }
            }
        }
        float corr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mnew[i] = fmaxf(mnew[i], __shfl_xor_sync(0xffffffffu, mnew[i], 1));
            mnew[i] = fmaxf(mnew[i], __shfl_xor_sync(0xffffffffu, mnew[i], 2));
            corr[i] = (mnew[i] == -INFINITY) ? 1.f : fast_exp2(mrow[i] - mnew[i]);
            mrow[i] = mnew[i];
            lrow[i] *= corr[i];
        }
        const float base[2] = {mnew[0] == -INFINITY ? 0.f : mnew[0], mnew[1] == -INFINITY ? 0.f : mnew[1]};
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = fast_exp2(s[j][e] - base[e >> 1]);   // 2^(-inf) = 0 for masked keys
                s[j][e] = pv;
                lrow[e >> 1] += pv;
            }
        }
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {   // no maximum moved: nothing to rescale
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < NK; ++kk) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dn = 0; dn < DV / 16; ++dn) {
                uint32_t vf[4];
                const int mat = lane >> 3, r = lane & 7;
                const __nv_bfloat16* vp = vst + (size_t)(key_off + kk * 16 + (mat & 1) * 8 + r) * LDV + dn * 16 + (mat >> 1) * 8;
                ldmatrix_x4_trans(vf, vp);
                mma_bf16(o[2 * dn], pf, vf[0], vf[1]);
                mma_bf16(o[2 * dn + 1], pf, vf[2], vf[3]);
            }
        }
        __syncthreads();
    }

    // each map's softmax: divide by the row's sum
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 1);
        lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 2);
    }
    float* other = reinterpret_cast<float*>(smem_raw);               // [rows of the tile][DV]: the second map's results
    if (SPLIT) {
        // the slabs' shares of the same 16 rows meet: [map][slab][row][DV values, maximum, sum] (the key and value stages
        // are done with); the first slab's warp of each map merges its map's four shares
        constexpr int RS = DV + 2;
        float* shares = reinterpret_cast<float*>(smem_raw);
        other = shares + 2 * 4 * 16 * RS;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float* dst = shares + (size_t)((map * 4 + rg) * 16 + gq + 8 * i) * RS;
#pragma unroll
            for (int dt = 0; dt < DV / 8; ++dt)
                *reinterpret_cast<float2*>(dst + dt * 8 + 2 * tq) = make_float2(o[dt][2 * i], o[dt][2 * i + 1]);
            if (tq == 0) {
                dst[DV] = mrow[i];
                dst[DV + 1] = lrow[i];
            }
        }
        __syncthreads();
        if (rg == 0) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float mx = -INFINITY;
                for (int g2 = 0; g2 < 4; ++g2) {
                    const float* src = shares + (size_t)((map * 4 + g2) * 16 + gq + 8 * i) * RS;
                    if (src[DV + 1] > 0.f) mx = fmaxf(mx, src[DV]);
                }
                float w[4];
                float total = 0.f;
                for (int g2 = 0; g2 < 4; ++g2) {                 // in the order of the slabs
                    const float* src = shares + (size_t)((map * 4 + g2) * 16 + gq + 8 * i) * RS;
                    w[g2] = src[DV + 1] > 0.f ? fast_exp2(src[DV] - mx) : 0.f;
                    total += src[DV + 1] * w[g2];
                }
                lrow[i] = total;
#pragma unroll
                for (int dt = 0; dt < DV / 8; ++dt) {
                    float a0 = 0.f, a1 = 0.f;
                    for (int g2 = 0; g2 < 4; ++g2) {
                        const float2 b = *reinterpret_cast<const float2*>(shares + (size_t)((map * 4 + g2) * 16 + gq + 8 * i) * RS + dt * 8 + 2 * tq);
                        a0 = fmaf(b.x, w[g2], a0);
                        a1 = fmaf(b.y, w[g2], a1);
                    }
                    o[dt][2 * i] = a0;
                    o[dt][2 * i + 1] = a1;
                }
            }
        }
    }
    const bool finishes = !SPLIT || rg == 0;                          // the warps that hold a map's whole result
    const float inv[2] = {lrow[0] > 0.f ? 1.f / lrow[0] : 0.f, lrow[1] > 0.f ? 1.f / lrow[1] : 0.f};
    // the second map's warps hand their results over in shared memory (the key and value stages are done with)
    if (map == 1 && finishes) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float* dst = other + (size_t)(row_base + gq + 8 * i) * DV;
#pragma unroll
            for (int dt = 0; dt < DV / 8; ++dt)
                *reinterpret_cast<float2*>(dst + dt * 8 + 2 * tq) = make_float2(o[dt][2 * i] * inv[i], o[dt][2 * i + 1] * inv[i]);
        }
    }
    __syncthreads();
    if (map == 1 || !finishes) return;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float* src = other + (size_t)(row_base + gq + 8 * i) * DV;
        float ss = 0.f;
#pragma unroll
        for (int dt = 0; dt < DV / 8; ++dt) {
            const float2 b = *reinterpret_cast<const float2*>(src + dt * 8 + 2 * tq);
            const float d0 = o[dt][2 * i] * inv[i] - p.lam * b.x, d1 = o[dt][2 * i + 1] * inv[i] - p.lam * b.y;
            o[dt][2 * i] = d0;
            o[dt][2 * i + 1] = d1;
            ss = fmaf(d0, d0, fmaf(d1, d1, ss));
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        if (!valid[i]) continue;
        const float rs = rsqrtf(ss / (float)DV + p.sub_eps) * p.out_scale;
        __nv_bfloat16* op = p.out + (size_t)tok[i] * p.out_stride + p.out_col + (size_t)head[i] * DV;
#pragma unroll
        for (int dt = 0; dt < DV / 8; ++dt)
            *reinterpret_cast<uint32_t*>(op + dt * 8 + 2 * tq) = pack_bf16(o[dt][2 * i] * rs, o[dt][2 * i + 1] * rs);
    }
}

template <int D, int DV, bool SPLIT>
cudaError_t launch_diff_as(const DiffParams& p, int n_tiles, cudaStream_t stream) {
    constexpr int WARPS = 8;
    static std::atomic<unsigned long long> done{0};
    constexpr int bytes_kv = (SPLIT ? 3 : 2) * (2 * KB * (D + 8) + KB * (DV + 8)) * 2;
    constexpr int bytes_out = SPLIT ? (2 * 4 * 16 * (DV + 2) + 16 * DV) * 4 : 16 * (WARPS / 2) * DV * 4;
    constexpr int bytes = bytes_kv > bytes_out ? bytes_kv : bytes_out;
    cudaError_t e = allow_dynamic_smem(attention_diff_kernel<D, DV, WARPS, SPLIT>, bytes, done);
    if (e != cudaSuccess) return e;
    return launch(attention_diff_kernel<D, DV, WARPS, SPLIT>, dim3(n_tiles, p.kv_heads), dim3(WARPS * 32), bytes, stream, p);
}

// A step of single tokens whose group of heads fits 16 rows: the slabs of warps share a block's keys, not the tile's rows.
template <int D, int DV>
cudaError_t launch_diff(const DiffParams& p, int n_tiles, cudaStream_t stream) {
    if (p.tiles == nullptr && p.heads / p.kv_heads <= 16) return launch_diff_as<D, DV, true>(p, n_tiles, stream);
    return launch_diff_as<D, DV, false>(p, n_tiles, stream);
}

}  // namespace

// rows (token, head of the group) of a tile
int attention_diff_tile_rows() { return 64; }

bool attention_diff_supports(int dim, int v_dim, int heads, int kv_heads) {
    if (kv_heads < 1 || heads % kv_heads || heads / kv_heads > attention_diff_tile_rows()) return false;
    return (dim == 32 && v_dim == 64) || (dim == 64 && v_dim == 128) || (dim == 128 && v_dim == 256) ||
           (dim == 64 && v_dim == 64) || (dim == 128 && v_dim == 128);
}

cudaError_t launch_attention_diff(const void* y, int y_stride, int q_col, void* out, int out_stride, int out_col, float out_scale,
                                  const void* k_cache, const void* v_cache, const int* cu_q, const int* q_start,
                                  const int* block_table, int table_stride, const int* tiles, int n_tiles, int tokens_per_tile,
                                  int n_pages, int heads, int kv_heads, int dim, int v_dim, int page_size, int window,
                                  int keep_first, float scale, float lam, float sub_eps, int* status, cudaStream_t stream) {
    if (n_tiles == 0) return cudaSuccess;
    if (!attention_diff_supports(dim, v_dim, heads, kv_heads) || page_size % 16) return cudaErrorInvalidValue;
    DiffParams p = {(const __nv_bfloat16*)y, y_stride, q_col, (__nv_bfloat16*)out, out_stride, out_col, out_scale,
                    (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, cu_q, q_start, block_table, table_stride,
                    reinterpret_cast<const int2*>(tiles), n_pages, heads, kv_heads, page_size, window, keep_first,
                    scale * 1.4426950408889634f, lam, sub_eps, tokens_per_tile, status};
    if (dim == 32 && v_dim == 64) return launch_diff<32, 64>(p, n_tiles, stream);
    if (dim == 64 && v_dim == 128) return launch_diff<64, 128>(p, n_tiles, stream);
    if (dim == 128 && v_dim == 256) return launch_diff<128, 256>(p, n_tiles, stream);
    if (dim == 64 && v_dim == 64) return launch_diff<64, 64>(p, n_tiles, stream);
    return launch_diff<128, 128>(p, n_tiles, stream);
}

}  // namespace vtb
