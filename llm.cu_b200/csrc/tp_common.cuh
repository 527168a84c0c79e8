// Layout of a tensor-parallel rank's exchange block (one cudaMalloc per rank, mapped into every peer through
// CUDA IPC; peers write into it over NVLink with plain stores, the owner polls it):
//
//   part 1, the whole-step kernel (decode_step.cu), one row per all-reduce
//     [0, 64)      flags[r]  u64: highest synchronisation number rank r has announced
//     [128, 144)   this rank's own counters (local, persist across launches)
//     [256, 512)   best[r]   (float value, int index): rank r's best logit of this step
//     [512, ...)   recv[2][tp][d_model] of (FP32 partial sum, 32-bit tag)
//     then         row[2][d_model / 2] of (two FP16 values, 32-bit tag): the all-reduced row, published locally
//   part 2, up to kTpRows rows at once (gemm_smallm.cu scatters, tp_rows.cu gathers)
//     rows_recv[2][tp][kTpRows][d_model] of (FP32 partial sum, 32-bit tag)
//     best_rows[tp][kTpRows][2] of (32-bit value, 32-bit tag): rank r's best (logit bits, global index) per row
//     seq          u32 (local): number of tagged exchanges completed so far; exchange j of a step carries
//                  the tag seq + j + 1, and the step's last kernel advances seq
//
// A value and its tag travel in one 8-byte store and a reader spins (bounded) until the tag is the one it
// expects, so no fence, flag or barrier stands between a producer and its consumers.
#pragma once

#include <stddef.h>

namespace llmb {

constexpr size_t kTpFlagsOff = 0, kTpBestOff = 256, kTpRecvOff = 512;
constexpr int kTpRows = 32;  // rows per exchange of the row-batched path (the N of the small-M projection)

__host__ __device__ constexpr size_t tp_row_off(int tp_size, int d) { return kTpRecvOff + (size_t)2 * tp_size * d * 8; }
__host__ __device__ constexpr size_t tp_step_bytes(int tp_size, int d) { return (tp_row_off(tp_size, d) + (size_t)2 * d * 4 + 255) / 256 * 256; }
__host__ __device__ constexpr size_t tp_rows_recv_off(int tp_size, int d) { return tp_step_bytes(tp_size, d); }
__host__ __device__ constexpr size_t tp_rows_recv_bytes(int tp_size, int d) { return (size_t)2 * tp_size * kTpRows * d * 8; }
__host__ __device__ constexpr size_t tp_rows_best_off(int tp_size, int d) { return tp_rows_recv_off(tp_size, d) + tp_rows_recv_bytes(tp_size, d); }
__host__ __device__ constexpr size_t tp_rows_seq_off(int tp_size, int d) { return tp_rows_best_off(tp_size, d) + (size_t)tp_size * kTpRows * 16; }
__host__ __device__ constexpr size_t tp_exchange_bytes(int tp_size, int d) { return tp_rows_seq_off(tp_size, d) + 256; }

// Where rank `src`'s partial sum of element (row b, column n) of exchange number `index` lands in a block.
__host__ __device__ inline size_t tp_rows_slot(int tp_size, int d, int index, int src, int b, int n) {
    return tp_rows_recv_off(tp_size, d) + ((((size_t)(index & 1) * tp_size + src) * kTpRows + b) * d + n) * 8;
}

}  // namespace llmb
