// Decode attention over the KV cache (one query row, grouped-query heads), split along the
// sequence ("flash-decode").
//
// Bound: HBM/L2 bandwidth on the cached K and V rows: algorithmic bytes per launch =
// (pos + 1) * 2 * n_kv_heads * head_dim * 2.  At the context lengths of the benchmark configs
// this is 1-4 % of a layer's weight bytes at batch 1 and a quarter of a step's bytes at 32 sequences:
// one pass, no N x N score buffer, and the arithmetic on the tensor cores so that a CTA is bound by its
// loads, not by instruction issue.
//
//   grid   (n_splits, n_kv_heads, n_seqs); CTA (s, g, b) handles cache rows [s*split_len, (s+1)*split_len)
//          of KV head g of sequence b for all `G` query heads of that group, so K and V are read once
//          per group, not once per query head.
//   block  128 threads = 4 warps; tiles of 64 cache rows in shared memory, two buffers: the next tile
//          streams in while this one is used, bytes counted on an mbarrier - as 64-row boxes through
//          tensor maps of the K and V cache (cp.async.bulk.tensor.2d, 128-byte swizzle) where the extent
//          of the cache is known (the batched entry point), else as one bulk copy per cache row and
//          thread into padded rows (cp.async.bulk).  Warp w takes keys 16w..16w+15 of every tile.  Tensor cores through mma.sync (m16n8k16, FP16 in, FP32 accumulate) with the KEYS as the
//          16 rows of the tile and the G query heads as its 8 columns: S^T = K q^T, scores /
//          sqrtf(head_dim) (inference.cu:784), online softmax in FP32 on the accumulator fragments,
//          O^T += V^T P^T with P split into an FP16 head and an FP16 remainder (two MMAs) so that the
//          probabilities enter the product with ~22 bits, as the reference's FP32 P does; P^T reaches
//          the operand layout with movmatrix.  24 MMAs per 16 keys (head_dim 128); with the heads as
//          rows of a 16-row tile it took 80 and the kernel was bound by the tensor pipe at 3 TB/s.
//          The four warps' (max, sum, out) meet in shared memory.
//   merge  each CTA writes (max, sum, unnormalised out) per query head to scratch; the last
//          CTA to finish for a (sequence, KV head) (atomic counter) rescales and adds the partials in
//          split order, normalises and writes FP16 (inference.cu:945).  The counter is left at zero.
//   batch  with several sequences the grid is not (split, head, sequence) but one wave of CTAs (as many
//          as are resident at once) in groups of n_kv_heads, one KV head per CTA.  The 64-row tiles of ALL
//          sequences are numbered sequence by sequence and shared evenly: group c takes tiles
//          [c*Q, (c+1)*Q) and so works on the tail of one sequence and the head of the next; a (sequence,
//          KV head)'s pieces are merged by the last of its CTAs to finish, in piece order.  Every CTA
//          streams the same number of bytes whatever the mix of sequence lengths, the per-CTA start-up
//          and merge cost is paid once per ~Q tiles, and the CTAs of a group ask for the same cache rows
//          (all KV heads of a row lie side by side) at the same time.
#include <mutex>

#include "gemm_common.cuh"
#include "mma_common.cuh"

namespace llmb {

constexpr int kAttnThreads = 128;
constexpr int kTile = 64;  // cache rows per shared-memory tile; two tiles take turns (one streams in while the other is used)

struct AttnParams {
    const __half *q;
    const __half *k_cache;
    const __half *v_cache;
    const int *pos;
    __half *out;
    int *counters;   // [n_kv_heads]
    float *part_ml;  // [n_kv_heads][n_splits][G][2]
    float *part_o;   // [n_kv_heads][n_splits][G][HD]
    int n_kv_heads, n_splits, split_len;
    // batched decode: blockIdx.z is the sequence; q and out are [n_seqs][n_q], pos is [n_seqs], the caches of
    // consecutive sequences are seq_stride elements apart (0 for a single sequence)
    int n_q;
    size_t seq_stride;
    unsigned long long *trace;  // optional profiling aid: [CTA][8] global-timer stamps (llmb_attn_decode_trace)
    int *status;                // device status word: a wait that runs out records its code there
    // balanced != 0 (several sequences): 1-D grid, tiles shared evenly; n_slots = n_splits + 1 partial slots per
    // (sequence, KV head); a piece is at least min_tiles tiles long
    int balanced, n_seqs, n_slots, min_tiles;
    int seq_rows;  // batched: cache rows per sequence (seq_stride = seq_rows * n_kv_heads * head_dim)
};

constexpr int kBalancedMaxSeqs = 256;

// A run of cache rows [begin, end) of one (sequence, KV head): what one CTA works on at a time.  Its partial goes
// to slot `slot` of the pair's partial slots; the last of the pair's n_used pieces to arrive merges them.
struct AttnPiece {
    int seq, g, begin, end, slot, n_used;
};

// Shared-memory image of a tile (64 cache rows of one KV head, K then V), two forms:
//  * rows: every row padded by 16 bytes, so that the 8 rows of an ldmatrix fall in distinct banks; filled by one
//    bulk copy per row and thread (the cache is only known as a pointer: the single-sequence entry points);
//  * boxes (TMA): the batched entry point knows the extent of the cache, so a tile is fetched as 64-row boxes of
//    128 bytes through a tensor map (one instruction per box instead of 128 row copies per tile, whose issue took
//    as long as the arithmetic), in the 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7).
template <int HD, bool TMA>
struct AttnTile {
    static constexpr int KP = HD + 8;
    static constexpr size_t kBytes = TMA ? (size_t)kTile * HD * 2 : (size_t)kTile * KP * 2;  // K or V part
    // byte offset of 16-byte chunk `chunk` of row `row` within the K (or V) part
    __device__ static __forceinline__ uint32_t off(int row, int chunk) {
        if (TMA) return (uint32_t)((chunk >> 3) * (kTile * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
        return (uint32_t)(row * KP * 2 + chunk * 16);
    }
};

// Requests tile i of a piece into buffer nth & 1 (`nth` counts all tiles the CTA has requested so far); completion
// is counted in bytes on the buffer's mbarrier.  Rows past the end of the piece: K rows there are masked after the
// product; V rows must be zero (0 * stale bits could be NaN): the row form zeroes them here, the box form after
// the tile has landed (attn_decode_segment).
template <int HD, bool TMA>
__device__ __forceinline__ void attn_request_tile(const AttnParams &p, const CUtensorMap *map_k, const CUtensorMap *map_v,
                                                  unsigned char *attn_smem, uint64_t *tile_bar, uint64_t policy, const AttnPiece &pc,
                                                  int i, uint32_t nth) {
    typedef AttnTile<HD, TMA> Tile;
    const int tid = threadIdx.x;
    const int buf = (int)(nth & 1u);
    unsigned char *kd = attn_smem + (size_t)buf * 2 * Tile::kBytes;
    unsigned char *vd = kd + Tile::kBytes;
    const int t0 = pc.begin + i * kTile;
    if (TMA) {
        if (tid == 0) {
            mbar_arrive_expect_tx(&tile_bar[buf], (uint32_t)(2 * Tile::kBytes));
            const int row = pc.seq * p.seq_rows + t0;  // row of the [n_seqs * seq_rows][n_kv_heads * HD] cache
#pragma unroll
            for (int b = 0; b < HD / 64; ++b) {
                tma_load_2d(kd + (size_t)b * kTile * 128, map_k, pc.g * HD + b * 64, row, &tile_bar[buf]);
                tma_load_2d(vd + (size_t)b * kTile * 128, map_v, pc.g * HD + b * 64, row, &tile_bar[buf]);
            }
        }
        return;
    }
    const int valid = min(kTile, pc.end - t0);
    if (tid == 0) mbar_arrive_expect_tx(&tile_bar[buf], (uint32_t)valid * HD * 2 * 2);
    const int r = tid & (kTile - 1);
    const bool v_row = tid >= kTile;
    if (r < valid) {
        const size_t goff = (size_t)pc.seq * p.seq_stride + (size_t)(t0 + r) * ((size_t)p.n_kv_heads * HD) + (size_t)pc.g * HD;
        bulk_g2s((v_row ? vd : kd) + Tile::off(r, 0), (v_row ? p.v_cache : p.k_cache) + goff, HD * 2, &tile_bar[buf], policy);
    } else if (v_row) {
#pragma unroll
        for (int ch = 0; ch < HD / 8; ++ch) *reinterpret_cast<uint4 *>(vd + Tile::off(r, ch)) = make_uint4(0u, 0u, 0u, 0u);
    }
}

// One piece.  `prefetched`: its first tile has been requested already (by the piece before it); `next`, if any,
// is the CTA's following piece: its first tile is requested while this piece's last tile is used, so that it
// streams in during this piece's publish and merge.
template <int HD, int G, bool TMA, typename Stamp>
__device__ __forceinline__ void attn_decode_segment(const AttnParams &p, const CUtensorMap *map_k, const CUtensorMap *map_v,
                                                    unsigned char *attn_smem, float (*wm_s)[8], float (*wl_s)[8],
                                                    int *is_last_s, uint64_t *tile_bar, uint32_t &tiles_before, uint64_t policy,
                                                    const AttnPiece &pc, bool prefetched, const AttnPiece *next, int n_slots,
                                                    Stamp stamp, long long &cyc_wait, long long &cyc_work) {
    const int seq = pc.seq, g = pc.g, begin = pc.begin, end = pc.end, slot = pc.slot, n_used = pc.n_used;
    static_assert(kAttnThreads == 2 * kTile, "one K row or one V row of a tile per thread");
    typedef AttnTile<HD, TMA> Tile;
    constexpr int KS = HD / 16;      // k-steps of q . k
    constexpr int MT = HD / 16;      // 16-dim row tiles of the output
    constexpr size_t kTileBytes = Tile::kBytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad_row = lane >> 2, quad_col = (lane & 3) * 2;
    int &is_last = *is_last_s;
    // the previous piece of this CTA is done with the shared memory; what it wrote there with ordinary stores is
    // ordered before the bulk copies that now overwrite it
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    const __half *q_seq = p.q + (size_t)seq * p.n_q + (size_t)g * G * HD;
    const int gs = seq * p.n_kv_heads + g;  // (sequence, KV head): index of the counter and of the partials
    static_assert(HD == 64 || HD == 128, "div_by_const is checked for sqrtf(64) and sqrtf(128)");
    const float sqrt_hd = sqrtf((float)HD), rsqrt_hd = __fdiv_rn(1.0f, sqrt_hd);

    // The keys are the rows of the MMA tile, the query heads its 8 columns (heads past G are zero columns):
    // S^T[16 keys][8 heads] = K[16 keys][HD] q^T, O^T[HD][8 heads] += V^T[HD][16 keys] P^T[16 keys][8 heads].
    // With the G heads as rows of a 16-row tile instead, three quarters of every MMA multiplied zeros, and the
    // kernel was bound by the warp-level tensor pipe, not by its loads.
    // B operand of K q^T: column quad_row is query head g * G + quad_row
    uint32_t qb[KS][2];
    {
        const bool real = quad_row < G;
        const __half *qr = q_seq + (size_t)(real ? quad_row : 0) * HD + quad_col;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qb[ks][0] = real ? *reinterpret_cast<const uint32_t *>(qr + ks * 16) : 0u;
            qb[ks][1] = real ? *reinterpret_cast<const uint32_t *>(qr + ks * 16 + 8) : 0u;
        }
    }
    // accumulator fragment: rows = dims mt*16 + quad_row (+8), columns = heads quad_col, quad_col + 1
    float o[MT][4];
#pragma unroll
    for (int t = 0; t < MT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f;
    // of heads quad_col and quad_col + 1, over this warp's keys (l: this lane's share)
    float m_run0 = -INFINITY, m_run1 = -INFINITY, l_run0 = 0.0f, l_run1 = 0.0f;

    const int n_tiles = end > begin ? (end - begin + kTile - 1) / kTile : 0;
    if (n_tiles > 0 && !prefetched) attn_request_tile<HD, TMA>(p, map_k, map_v, attn_smem, tile_bar, policy, pc, 0, tiles_before);
    for (int ti = 0; ti < n_tiles; ++ti) {
        // the next tile (of this piece, or the first one of the next piece) streams in while this one is used
        if (ti + 1 < n_tiles)
            attn_request_tile<HD, TMA>(p, map_k, map_v, attn_smem, tile_bar, policy, pc, ti + 1, tiles_before + (uint32_t)ti + 1u);
        else if (next)
            attn_request_tile<HD, TMA>(p, map_k, map_v, attn_smem, tile_bar, policy, *next, 0, tiles_before + (uint32_t)n_tiles);
        const uint32_t nth = tiles_before + (uint32_t)ti;
        const long long c0 = p.trace ? clock64() : 0;
        mbar_wait_warp(&tile_bar[nth & 1u], (nth >> 1) & 1u, p.status, 331, lane);
        const long long c1 = p.trace ? clock64() : 0;
        unsigned char *k_s = attn_smem + (size_t)(nth & 1u) * 2 * kTileBytes;
        unsigned char *v_s = k_s + kTileBytes;
        if (begin + (ti + 1) * kTile > end) {  // a ragged tile: V rows past the end are zero
            if (TMA) {
                const int valid = end - (begin + ti * kTile);
                for (int idx = tid; idx < (kTile - valid) * (HD / 8); idx += kAttnThreads)
                    *reinterpret_cast<uint4 *>(v_s + Tile::off(valid + idx / (HD / 8), idx % (HD / 8))) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncthreads();  // the zeroed rows are other threads' stores
        }
        if (ti == 0) stamp(2);
        const int key0 = begin + ti * kTile + warp * 16;  // this warp's 16 keys of the tile
        if (key0 < end) {
            // S^T = K q^T: A fragments of the 16 key rows through ldmatrix
            float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // (key quad_row, heads quad_col, +1), (key quad_row + 8, same heads)
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t ka[4];
                ldmatrix_x4(ka, k_s + Tile::off(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
                mma_16816(sc, ka, qb[ks][0], qb[ks][1]);
            }
            // scale (inference.cu:784), mask keys past the end, maximum per head over the 16 keys
            // (the columns past G hold exact zeros: they are not divided - an IEEE division of zero leaves the
            // fast path, and with half or more of the lanes doing so it was most of this kernel's time - and
            // keep the score 0, which stays finite through the softmax)
            const bool in_a = key0 + quad_row < end, in_b = key0 + quad_row + 8 < end;
            const bool real0 = quad_col < G, real1 = quad_col + 1 < G;
            sc[0] = real0 ? (in_a ? div_by_const(sc[0], sqrt_hd, rsqrt_hd) : -INFINITY) : 0.0f;
            sc[1] = real1 ? (in_a ? div_by_const(sc[1], sqrt_hd, rsqrt_hd) : -INFINITY) : 0.0f;
            sc[2] = real0 ? (in_b ? div_by_const(sc[2], sqrt_hd, rsqrt_hd) : -INFINITY) : 0.0f;
            sc[3] = real1 ? (in_b ? div_by_const(sc[3], sqrt_hd, rsqrt_hd) : -INFINITY) : 0.0f;
            float tm0 = fmaxf(sc[0], sc[2]), tm1 = fmaxf(sc[1], sc[3]);
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, off));
                tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, off));
            }
            const float m_new0 = fmaxf(m_run0, tm0), m_new1 = fmaxf(m_run1, tm1);  // finite: key0 < end
            const float scale0 = (m_run0 == -INFINITY) ? 0.0f : expf(m_run0 - m_new0);
            const float scale1 = (m_run1 == -INFINITY) ? 0.0f : expf(m_run1 - m_new1);
            m_run0 = m_new0;
            m_run1 = m_new1;
            l_run0 *= scale0;
            l_run1 *= scale1;
#pragma unroll
            for (int t = 0; t < MT; ++t) {
                o[t][0] *= scale0;
                o[t][1] *= scale1;
                o[t][2] *= scale0;
                o[t][3] *= scale1;
            }
            // probabilities: an FP16 head and an FP16 remainder (two MMAs), so that they enter the product with
            // ~22 bits, as the reference's FP32 probabilities do; exp(-inf) = 0 for masked keys
            const float p0 = expf(sc[0] - m_new0), p1 = expf(sc[1] - m_new1), p2 = expf(sc[2] - m_new0), p3 = expf(sc[3] - m_new1);
            l_run0 += p0 + p2;
            l_run1 += p1 + p3;
            const __half2 h01 = __floats2half2_rn(p0, p1), h23 = __floats2half2_rn(p2, p3);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            // P^T as the B operand wants (keys 2t, 2t+1 | head quad_row): the transpose of what the accumulator holds
            const uint32_t pb_hi0 = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&h01));
            const uint32_t pb_hi1 = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&h23));
            const uint32_t pb_lo0 = movmatrix_trans(pack_half2(p0 - f01.x, p1 - f01.y));
            const uint32_t pb_lo1 = movmatrix_trans(pack_half2(p2 - f23.x, p3 - f23.y));
            // O^T += V^T P^T: A fragments of V^T through ldmatrix.trans (V rows are keys)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t va[4];
                ldmatrix_x4_trans(va, v_s + Tile::off(warp * 16 + (lane & 7) + (lane >> 4) * 8, mt * 2 + ((lane >> 3) & 1)));
                mma_16816(o[mt], va, pb_hi0, pb_hi1);
                mma_16816(o[mt], va, pb_lo0, pb_lo1);
            }
        }
        __syncthreads();  // this tile's buffer is free for the tile after next
        if (p.trace) {
            cyc_wait += c1 - c0;
            cyc_work += clock64() - c1;
        }
    }
    tiles_before += (uint32_t)n_tiles;

    stamp(3);
    // ---- the four warps' states meet in shared memory (the tile buffers are idle now) ----
    // (the buffer of this piece's last tile is idle now; the other one may be receiving the next piece's first tile)
    unsigned char *idle_buf = attn_smem + (size_t)((tiles_before - 1u) & 1u) * 2 * kTileBytes;
    float *wo_s = reinterpret_cast<float *>(idle_buf);  // [4 warps][G][HD]
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        l_run0 += __shfl_xor_sync(0xffffffffu, l_run0, off);
        l_run1 += __shfl_xor_sync(0xffffffffu, l_run1, off);
    }
    if (quad_col < G) {
        if (quad_row == 0) {
            wm_s[warp][quad_col] = m_run0;
            wl_s[warp][quad_col] = l_run0;
        }
#pragma unroll
        for (int t = 0; t < MT; ++t) {
            wo_s[((size_t)warp * G + quad_col) * HD + t * 16 + quad_row] = o[t][0];
            wo_s[((size_t)warp * G + quad_col) * HD + t * 16 + quad_row + 8] = o[t][2];
        }
    }
    if (quad_col + 1 < G) {
        if (quad_row == 0) {
            wm_s[warp][quad_col + 1] = m_run1;
            wl_s[warp][quad_col + 1] = l_run1;
        }
#pragma unroll
        for (int t = 0; t < MT; ++t) {
            wo_s[((size_t)warp * G + quad_col + 1) * HD + t * 16 + quad_row] = o[t][1];
            wo_s[((size_t)warp * G + quad_col + 1) * HD + t * 16 + quad_row + 8] = o[t][3];
        }
    }
    __syncthreads();
    // CTA partial of (head h, dim d): warps combined in warp order.  A pair that is a single piece is finished
    // here (the merge of one piece is the identity: weight expf(0) = 1), without the trip through scratch.
    const size_t pbase = ((size_t)gs * n_slots + slot) * G;
    for (int e = tid; e < G * HD; e += kAttnThreads) {
        const int h = e / HD, dd = e % HD;
        const float M = fmaxf(fmaxf(wm_s[0][h], wm_s[1][h]), fmaxf(wm_s[2][h], wm_s[3][h]));
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float wgt = (wm_s[w][h] == -INFINITY) ? 0.0f : expf(wm_s[w][h] - M);
            num = fmaf(wgt, wo_s[((size_t)w * G + h) * HD + dd], num);
            den = fmaf(wgt, wl_s[w][h], den);
        }
        if (n_used == 1) {
            p.out[(size_t)seq * p.n_q + ((size_t)g * G + h) * HD + dd] = __float2half_rn(__fdiv_rn(fmaf(1.0f, num, 0.0f), fmaf(1.0f, den, 0.0f)));
            continue;
        }
        p.part_o[(pbase + h) * HD + dd] = num;
        if (dd == 0) {
            p.part_ml[(pbase + h) * 2] = M;
            p.part_ml[(pbase + h) * 2 + 1] = den;
        }
    }
    if (n_used == 1) {
        stamp(4);
        return;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(&p.counters[gs], 1);
        is_last = (prev == n_used - 1);
        if (is_last) p.counters[gs] = 0;  // every split in use has arrived; ready for the next launch
    }
    __syncthreads();
    stamp(4);
    if (!is_last) return;
    __threadfence();

    // Merge, in piece order.  One round of loads: the (max, sum) pairs of all pieces and, for every output element of
    // this thread, the partial outputs of the first four pieces; the sums themselves stay in piece order.
    constexpr int EPT = (G * HD + kAttnThreads - 1) / kAttnThreads;  // output elements per thread
    const size_t gbase = (size_t)gs * n_slots * G;
    float o4[EPT][4];
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = tid + j * kAttnThreads;
        const float *po = p.part_o + (gbase + (size_t)(e / HD)) * HD + (e % HD);
#pragma unroll
        for (int i = 0; i < 4; ++i) o4[j][i] = (e < G * HD && i < n_used) ? __ldcg(po + (size_t)i * G * HD) : 0.0f;
    }
    float *mg_m = reinterpret_cast<float *>(idle_buf);  // [n_used][G] maxima, then weights
    float *mg_l = mg_m + (size_t)n_used * G;            // [n_used][G] sums
    float *mg_den = mg_l + (size_t)n_used * G;          // [G]
    for (int i = tid; i < n_used * G; i += kAttnThreads) {
        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(p.part_ml) + gbase + i);
        mg_m[i] = ml.x;
        mg_l[i] = ml.y;
    }
    __syncthreads();
    if (tid < G) {
        float M = -INFINITY;
        for (int sidx = 0; sidx < n_used; ++sidx) M = fmaxf(M, mg_m[sidx * G + tid]);
        float den = 0.0f;
        for (int sidx = 0; sidx < n_used; ++sidx) {
            const float m = mg_m[sidx * G + tid];
            const float wgt = (m == -INFINITY) ? 0.0f : expf(m - M);
            den = fmaf(wgt, mg_l[sidx * G + tid], den);
            mg_m[sidx * G + tid] = wgt;
        }
        mg_den[tid] = den;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = tid + j * kAttnThreads;
        if (e < G * HD) {
            const int head = e / HD, dd = e % HD;
            const float *po = p.part_o + (gbase + head) * HD + dd;
            float num = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i < n_used) num = fmaf(mg_m[i * G + head], o4[j][i], num);
            for (int sidx = 4; sidx < n_used; ++sidx) num = fmaf(mg_m[sidx * G + head], __ldcg(po + (size_t)sidx * G * HD), num);
            p.out[(size_t)seq * p.n_q + ((size_t)g * G + head) * HD + dd] = __float2half_rn(__fdiv_rn(num, mg_den[head]));
        }
    }
    stamp(5);
}

template <int HD, int G, bool TMA>
__global__ void __launch_bounds__(kAttnThreads, 3)
attn_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    static_assert(G <= 8, "the query heads of a KV head are the columns of one 8-column MMA tile");
    extern __shared__ __align__(16) unsigned char attn_smem_raw[];
    // the swizzled boxes want 1024-byte alignment
    unsigned char *attn_smem =
        TMA ? reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(attn_smem_raw) + 1023) & ~uintptr_t(1023)) : attn_smem_raw;
    __shared__ float wm_s[4][8], wl_s[4][8];  // per warp and query head: running maximum and sum
    __shared__ int is_last;
    __shared__ __align__(8) uint64_t tile_bar[2];  // bytes landed in each of the two tile buffers
    __shared__ int pre_s[kBalancedMaxSeqs + 1];  // balanced: tiles of the sequences before each sequence
    __shared__ int len_s[kBalancedMaxSeqs];
    __shared__ int longest_s;

    const int tid = threadIdx.x;
    const size_t cta = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    auto stamp = [&](int which) {
        if (p.trace && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t) :: "memory");
            p.trace[cta * 8 + which] = t;
        }
    };
    stamp(0);
    pdl_launch_dependents();
    if (tid == 0) {
        mbar_init(&tile_bar[0], 1);
        mbar_init(&tile_bar[1], 1);
        fence_mbar_init();
    }
    __syncthreads();
    uint32_t tiles_before = 0;  // tiles this CTA has requested so far: buffer and mbarrier phase of the next one
    long long cyc_wait = 0, cyc_work = 0;  // trace only: SM cycles of thread 0 spent waiting for tiles / using them
    const uint64_t policy = policy_evict_first();
    pdl_wait();
    stamp(1);

    if (!p.balanced) {
        const int split = blockIdx.x, g = blockIdx.y, seq = blockIdx.z;
        const int len_total = p.pos[seq] + 1;
        const int begin = split * p.split_len;
        // a split that starts past the sequence has nothing to add: the merge only waits for the splits in use
        if (begin >= len_total) return;
        const AttnPiece pc = {seq, g, begin, min(begin + p.split_len, len_total), split,
                              min(p.n_splits, (len_total + p.split_len - 1) / p.split_len)};
        attn_decode_segment<HD, G, TMA>(p, &map_k, &map_v, attn_smem, wm_s, wl_s, &is_last, tile_bar, tiles_before, policy, pc, false, nullptr, p.n_slots,
                                   stamp, cyc_wait, cyc_work);
        if (p.trace && tid == 0) {
            p.trace[cta * 8 + 6] = (unsigned long long)cyc_wait;
            p.trace[cta * 8 + 7] = (unsigned long long)cyc_work;
        }
        return;
    }

    // ---- balanced: the tiles of all (sequence, KV head) pairs, numbered pair by pair, in equal shares ----
    for (int sq = tid; sq < p.n_seqs; sq += kAttnThreads) {  // one round of loads for all sequences
        const int len = p.pos[sq] + 1;
        len_s[sq] = len;
        pre_s[sq + 1] = (len + kTile - 1) / kTile;
    }
    __syncthreads();
    if (tid < 32) {  // inclusive scan of up to 256 tile counts: 8 per lane, then across the warp
        int v[8], sum = 0, longest = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = tid * 8 + i;
            v[i] = idx < p.n_seqs ? pre_s[idx + 1] : 0;
            sum += v[i];
            longest = max(longest, v[i]);
        }
        int incl = sum;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, off);
            if (tid >= off) incl += up;
            longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, off));
        }
        int run = incl - sum;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = tid * 8 + i;
            run += v[i];
            if (idx < p.n_seqs) pre_s[idx + 1] = run;
        }
        if (tid == 0) {
            pre_s[0] = 0;
            longest_s = longest;
        }
    }
    __syncthreads();
    const int longest = longest_s;
    // n_kv_heads consecutive CTAs form a group that walks the same run of tiles, one KV head each: a cache row
    // holds all KV heads side by side, so the group's requests for a row arrive together and the row is fetched
    // from DRAM in one piece.  The groups share the tiles of all sequences, numbered sequence by sequence, evenly.
    const int groups = (int)gridDim.x / p.n_kv_heads;
    const int g = (int)blockIdx.x % p.n_kv_heads, grp = (int)blockIdx.x / p.n_kv_heads;
    if (grp >= groups) return;
    const int total = pre_s[p.n_seqs];
    // quota: an equal share, but pieces no shorter than asked and never more than n_slots pieces per sequence
    // (a sequence of T tiles meets at most ceil(T / Q) + 1 groups, and Q >= ceil(longest / n_splits))
    int quota = (total + groups - 1) / groups;
    quota = max(quota, max(p.min_tiles, (longest + p.n_splits - 1) / p.n_splits));
    const int t_end = min((grp + 1) * quota, total);
    // the piece that starts at tile t of the group's run (t < t_end)
    auto piece_at = [&](int t, int &seq, int &tiles) {
        while (pre_s[seq + 1] <= t) ++seq;
        const int t_seq = pre_s[seq + 1] - pre_s[seq];  // tiles of this sequence
        const int j0 = t - pre_s[seq];
        const int j1 = min(t_seq, j0 + (t_end - t));
        const int first_grp = pre_s[seq] / quota, last_grp = (pre_s[seq + 1] - 1) / quota;
        tiles = j1 - j0;
        return AttnPiece{seq, g, j0 * kTile, min(j1 * kTile, len_s[seq]), grp - first_grp, last_grp - first_grp + 1};
    };
    int t = grp * quota;
    if (t >= t_end) return;
    int seq = 0, tiles = 0;
    AttnPiece pc = piece_at(t, seq, tiles);
    bool prefetched = false;
    for (;;) {
        t += tiles;
        const bool more = t < t_end;
        AttnPiece nxt = pc;
        int next_tiles = 0;
        if (more) nxt = piece_at(t, seq, next_tiles);
        attn_decode_segment<HD, G, TMA>(p, &map_k, &map_v, attn_smem, wm_s, wl_s, &is_last, tile_bar, tiles_before, policy, pc, prefetched,
                                   more ? &nxt : nullptr, p.n_slots, stamp, cyc_wait, cyc_work);
        if (p.trace && tid == 0) {
            p.trace[cta * 8 + 6] = (unsigned long long)cyc_wait;
            p.trace[cta * 8 + 7] = (unsigned long long)cyc_work;
        }
        if (!more) break;
        pc = nxt;
        tiles = next_tiles;
        prefetched = true;
    }
}

template <int HD, int G, bool TMA>
static int launch_attn_form(const AttnParams &p, const CUtensorMap &mk, const CUtensorMap &mv, int n_seqs, bool pdl, cudaStream_t stream) {
    // two buffers of (K tile, V tile): 64 padded rows each, or swizzled boxes (1024-byte aligned)
    const size_t smem = 4 * AttnTile<HD, TMA>::kBytes + (TMA ? 1024 : 0);
    static size_t attr_set[kMaxDevices] = {};  // per instantiation and device
    LLMB_CUDA_OK(ensure_dynamic_smem(attn_decode_kernel<HD, G, TMA>, attr_set, smem));
    dim3 grid(p.n_splits, p.n_kv_heads, n_seqs);
    if (p.balanced) {
        // one wave: as many CTAs as are resident at once (the kernel gives each an equal share of the tiles)
        static int resident[kMaxDevices] = {};
        const int slot = current_device_slot();
        if (slot < 0) return LLMB_ERR_CUDA;
        if (!resident[slot]) {
            int per_sm = 0;
            LLMB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_kernel<HD, G, TMA>, kAttnThreads, smem));
            resident[slot] = (per_sm > 0 ? per_sm : 1) * sm_count_cached();
        }
        // whole groups of n_kv_heads CTAs (at least one)
        const int groups = resident[slot] / p.n_kv_heads > 0 ? resident[slot] / p.n_kv_heads : 1;
        grid = dim3(groups * p.n_kv_heads, 1, 1);
    }
    LLMB_CUDA_OK(launch_pdl(attn_decode_kernel<HD, G, TMA>, grid, dim3(kAttnThreads), smem, stream, pdl, mk, mv, p));
    return LLMB_OK;
}

// The batched entry point knows the extent of the cache (n_seqs * seq_rows rows): tiles then come through tensor
// maps of the K and the V cache of the layer; otherwise row by row.
template <int HD, int G>
static int launch_attn(const AttnParams &p, int n_seqs, bool pdl, cudaStream_t stream) {
    CUtensorMap mk = {}, mv = {};
    if (p.seq_rows > 0 && (long long)n_seqs * p.seq_rows < (1ll << 31) && (((uintptr_t)p.k_cache | (uintptr_t)p.v_cache) & 15) == 0) {
        int rc;
        if ((rc = make_map(&mk, p.k_cache, n_seqs * p.seq_rows, p.n_kv_heads * HD, kTile))) return rc;
        if ((rc = make_map(&mv, p.v_cache, n_seqs * p.seq_rows, p.n_kv_heads * HD, kTile))) return rc;
        return launch_attn_form<HD, G, true>(p, mk, mv, n_seqs, pdl, stream);
    }
    return launch_attn_form<HD, G, false>(p, mk, mv, n_seqs, pdl, stream);
}

static size_t attn_counters_bytes(int n_kv_heads) { return ((size_t)n_kv_heads * 4 + 255) / 256 * 256; }

}  // namespace llmb

extern "C" size_t llmb_attn_decode_scratch_bytes(int n_q_heads, int n_kv_heads, int head_dim, int n_splits) {
    if (n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || n_splits <= 0) return 0;
    size_t ml = ((size_t)n_q_heads * n_splits * 2 * 4 + 255) / 256 * 256;
    size_t o = (size_t)n_q_heads * n_splits * head_dim * 4;
    return llmb::attn_counters_bytes(n_kv_heads) + ml + o;
}

static unsigned long long *g_attn_trace = nullptr;

// Profiling aid: per-CTA global-timer stamps of the next launches (entry, previous kernel complete, first tile
// landed, tiles done, partial published, merge done - of the CTA's last piece), then the SM cycles thread 0 spent
// waiting for tiles and using them (all pieces), into a device buffer of 8 uint64 per CTA; NULL turns it off.
extern "C" int llmb_attn_decode_trace(void *d_trace) {
    g_attn_trace = static_cast<unsigned long long *>(d_trace);
    return LLMB_OK;
}

static int attn_decode_impl(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache, const int32_t *d_pos,
                            int n_seqs, size_t seq_stride_elems, int n_q_heads, int n_kv_heads, int head_dim, int n_splits,
                            int split_len, uint16_t *d_out, void *d_scratch, int use_pdl, llmb_stream_t stream_,
                            bool batch_scratch = false) {
    using namespace llmb;
    if (!d_q || !d_k_cache || !d_v_cache || !d_pos || !d_out || !d_scratch) return LLMB_ERR_INVALID;
    if (n_kv_heads <= 0 || n_q_heads % n_kv_heads || n_splits <= 0 || split_len <= 0 || n_seqs <= 0 || n_seqs > 65535)
        return LLMB_ERR_INVALID;
    if (((uintptr_t)d_scratch & 255) || ((uintptr_t)d_k_cache & 15) || ((uintptr_t)d_v_cache & 15) || (seq_stride_elems & 7))
        return LLMB_ERR_INVALID;
    AttnParams p;
    p.q = reinterpret_cast<const __half *>(d_q);
    p.k_cache = reinterpret_cast<const __half *>(d_k_cache);
    p.v_cache = reinterpret_cast<const __half *>(d_v_cache);
    p.pos = d_pos;
    p.out = reinterpret_cast<__half *>(d_out);
    // scratch of n_seqs sequences = the layout of one sequence with n_seqs times the heads
    unsigned char *sc = static_cast<unsigned char *>(d_scratch);
    // several sequences: tiles shared evenly over one wave of CTAs, one more partial slot per pair than splits
    p.balanced = (n_seqs > 1 && n_seqs <= kBalancedMaxSeqs) ? 1 : 0;
    p.n_seqs = n_seqs;
    p.n_slots = n_splits + (batch_scratch ? 1 : 0);
    p.min_tiles = split_len / kTile > 0 ? split_len / kTile : 1;
    if (p.balanced && !batch_scratch) p.balanced = 0;
    p.counters = reinterpret_cast<int *>(sc);
    sc += attn_counters_bytes(n_kv_heads * n_seqs);
    p.part_ml = reinterpret_cast<float *>(sc);
    sc += ((size_t)n_q_heads * n_seqs * p.n_slots * 2 * 4 + 255) / 256 * 256;
    p.part_o = reinterpret_cast<float *>(sc);
    p.n_kv_heads = n_kv_heads;
    p.n_splits = n_splits;
    p.split_len = split_len;
    p.n_q = n_q_heads * head_dim;
    p.seq_stride = seq_stride_elems;
    p.seq_rows = batch_scratch ? (int)(seq_stride_elems / ((size_t)n_kv_heads * head_dim)) : 0;
    p.trace = g_attn_trace;
    p.status = device_status_ptr();
    if (!p.status) return LLMB_ERR_CUDA;
    const int G = n_q_heads / n_kv_heads;
    const bool pdl = use_pdl != 0;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (head_dim == 128) {
        switch (G) {
            case 1: return launch_attn<128, 1>(p, n_seqs, pdl, stream);
            case 2: return launch_attn<128, 2>(p, n_seqs, pdl, stream);
            case 4: return launch_attn<128, 4>(p, n_seqs, pdl, stream);
            case 8: return launch_attn<128, 8>(p, n_seqs, pdl, stream);
        }
    } else if (head_dim == 64) {
        switch (G) {
            case 2: return launch_attn<64, 2>(p, n_seqs, pdl, stream);
            case 4: return launch_attn<64, 4>(p, n_seqs, pdl, stream);
            case 8: return launch_attn<64, 8>(p, n_seqs, pdl, stream);
        }
    }
    return LLMB_ERR_UNSUPPORTED;
}

extern "C" int llmb_attn_decode(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache,
                                const int32_t *d_pos, int n_q_heads, int n_kv_heads, int head_dim, int n_splits,
                                int split_len, uint16_t *d_out, void *d_scratch, int use_pdl, llmb_stream_t stream_) {
    return attn_decode_impl(d_q, d_k_cache, d_v_cache, d_pos, 1, 0, n_q_heads, n_kv_heads, head_dim, n_splits, split_len, d_out,
                            d_scratch, use_pdl, stream_);
}

extern "C" size_t llmb_attn_decode_batch_scratch_bytes(int n_seqs, int n_q_heads, int n_kv_heads, int head_dim, int n_splits) {
    if (n_seqs <= 0 || n_splits <= 0) return 0;
    // one slot more than splits per (sequence, KV head): a pair's tiles can straddle one more CTA than its share
    return llmb_attn_decode_scratch_bytes(n_q_heads * n_seqs, n_kv_heads * n_seqs, head_dim, n_splits + 1);
}

extern "C" int llmb_attn_decode_batch(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache,
                                      const int32_t *d_pos, int n_seqs, size_t seq_stride_rows, int n_q_heads, int n_kv_heads,
                                      int head_dim, int n_splits, int split_len, uint16_t *d_out, void *d_scratch, int use_pdl,
                                      llmb_stream_t stream_) {
    if (n_kv_heads <= 0 || head_dim <= 0) return LLMB_ERR_INVALID;
    return attn_decode_impl(d_q, d_k_cache, d_v_cache, d_pos, n_seqs, seq_stride_rows * (size_t)n_kv_heads * head_dim, n_q_heads,
                            n_kv_heads, head_dim, n_splits, split_len, d_out, d_scratch, use_pdl, stream_, true);
}

// ---------------------------------------------------------------------------------------
// llmb_attn_decode_static: the same split-KV attention, for hosts that must not allocate.
//
// Some programs that embed this library cannot call cudaMalloc themselves: an inference
// server that handed the whole device to its own pool at start-up and treats any later
// driver allocation as a bug, a real-time loop that cannot take the device-wide
// synchronisation an allocation may imply, or a plug-in that only receives input and output
// buffers from its host and has nowhere to keep a workspace.  For them the partial results
// live in the fixed array below instead of a caller-provided workspace.
//
//  * Limit: n_q_heads * n_splits <= 4096, head_dim <= 128, n_kv_heads <= 64; the array is
//    2,130,176 bytes and every GPU that loads the library carries it until the process ends.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress:
//    in host code the array's name is only a handle, not something a kernel can dereference)
//    and remembers it; make that first call before starting any stream capture.  If the
//    library's device code has not been loaded on that device yet, this look-up is what makes
//    the CUDA runtime load it (the array and the kernels then take their place in device
//    memory), so make the first call at start-up, not inside the allocation-free region.
//  * All calls on a device share the one array and it keeps whatever the previous call
//    left, so the arrival counters are cleared on the stream before each launch; two calls
//    that can overlap on the GPU (different streams, no dependency) race on it.
//  * No cudaMalloc, cudaFree or allocating library routine is called.
// ---------------------------------------------------------------------------------------
namespace llmb {

constexpr int kStaticMaxHeadSplits = 4096;  // n_q_heads * n_splits
constexpr int kStaticMaxHeadDim = 128;
constexpr int kStaticMaxKvHeads = 64;
constexpr size_t kStaticCounterBytes = 256;
constexpr size_t kStaticMlBytes = (size_t)kStaticMaxHeadSplits * 2 * sizeof(float);
constexpr size_t kStaticScratchBytes =
    kStaticCounterBytes + kStaticMlBytes + (size_t)kStaticMaxHeadSplits * kStaticMaxHeadDim * sizeof(float);

static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

static std::mutex g_static_mu;
static void *g_static_ptr[64] = {};

// Device address of the array on the current device (looked up once per device).
static int static_scratch_ptr(void **out) {
    int dev = 0;
    LLMB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_last_error("llmb_attn_decode_static: device ordinal above 63");
        return LLMB_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
        void *ptr = nullptr;
        LLMB_CUDA_OK(cudaGetSymbolAddress(&ptr, g_attn_static_scratch));
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return LLMB_OK;
}

}  // namespace llmb

extern "C" int llmb_attn_decode_static(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache,
                                       const int32_t *d_pos, int n_q_heads, int n_kv_heads, int head_dim, int n_splits,
                                       int split_len, uint16_t *d_out, int use_pdl, llmb_stream_t stream_) {
    using namespace llmb;
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_splits <= 0 || head_dim <= 0) return LLMB_ERR_INVALID;
    if ((long long)n_q_heads * n_splits > kStaticMaxHeadSplits || head_dim > kStaticMaxHeadDim ||
        n_kv_heads > kStaticMaxKvHeads) {
        set_last_error(
            "llmb_attn_decode_static: request exceeds the built-in workspace (n_q_heads * n_splits <= 4096, "
            "head_dim <= 128, n_kv_heads <= 64); use llmb_attn_decode with a caller-provided workspace");
        return LLMB_ERR_UNSUPPORTED;
    }
    // the argument checks llmb_attn_decode makes, here already: nothing is queued on the stream for a call
    // that is going to be refused
    if (!d_q || !d_k_cache || !d_v_cache || !d_pos || !d_out) return LLMB_ERR_INVALID;
    if (split_len <= 0 || n_q_heads % n_kv_heads) return LLMB_ERR_INVALID;
    if (((uintptr_t)d_k_cache & 15) || ((uintptr_t)d_v_cache & 15)) return LLMB_ERR_INVALID;
    void *scratch = nullptr;
    int rc = static_scratch_ptr(&scratch);
    if (rc) return rc;
    // Carve the array exactly as llmb_attn_decode carves a caller workspace of this request's size:
    // the layout depends on the request, not on the array's capacity, and fits by the check above.
    if (llmb_attn_decode_scratch_bytes(n_q_heads, n_kv_heads, head_dim, n_splits) > kStaticScratchBytes) {
        set_last_error("llmb_attn_decode_static: request exceeds the built-in workspace");
        return LLMB_ERR_UNSUPPORTED;
    }
    // The counters must start at zero; a finished call leaves them so, an interrupted one may not.
    LLMB_CUDA_OK(cudaMemsetAsync(scratch, 0, kStaticCounterBytes, static_cast<cudaStream_t>(stream_)));
    return llmb_attn_decode(d_q, d_k_cache, d_v_cache, d_pos, n_q_heads, n_kv_heads, head_dim, n_splits, split_len,
                            d_out, scratch, use_pdl, stream_);
}
