// Pieces shared by the tensor-core projection kernels (gemm_tc.cu: blocks of rows; gemm_smallm.cu: a handful of
// rows with the weights as the 128-row operand): tile constants, the parameter block, tcgen05 / TMA wrappers
// and the host-side tensor-map builder.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace llmb {

constexpr int kBM = 128, kBK = 64;
constexpr int kGemmThreads = 192;
constexpr uint32_t kATileBytes = kBM * kBK * 2;  // 16 KB: the A tile of a stage
constexpr int kGemmMaxStages = 8;
// Ring depth: two CTAs share an SM when the grid has more CTAs than SMs (3 stages each, 2 for SwiGLU);
// a grid that leaves every CTA alone on its SM gets a ring as deep as shared memory allows, because
// then the copy latency is hidden by nothing but the ring.
__host__ __device__ constexpr int gemm_stages(bool dual) { return dual ? 2 : 3; }
__host__ __device__ constexpr uint32_t gemm_stage_bytes(bool dual, int bn) { return kATileBytes + (dual ? 2 : 1) * bn * kBK * 2; }

struct GemmParams {
    __half *c;              // STORE/RESIDUAL/SWIGLU: [M][N] (SWIGLU: N = ffn); ROPE_KV: q [M][n_q]
    const float2 *rope_cs;  // ROPE_KV: [M][head_dim / 2]
    __half *k_cache, *v_cache;
    int *status;
    int M, N, K, epilogue;
    int n_q, n_kv, head_dim, pos0, max_pos;
    const int *row_pos;  // ROPE_KV, batched decode: cache position of each row; row r belongs to sequence r
    long long seq_stride;  // cache rows between consecutive sequences
    int stages;  // ring depth of this launch (<= kGemmMaxStages)
    // split-K: blockIdx.z takes a slice of K, partial accumulators meet in the workspace and the last
    // CTA of a tile to arrive adds them in slice order and runs the epilogue
    int splits;
    float *ws_part;  // [tiles][splits][128][accumulator columns]
    int *ws_count;   // [tiles], zero between launches
    // LLMB_EPI_TP_SCATTER (small-M kernel): the output is this rank's partial sum of a row-parallel projection;
    // it goes, tagged, into every rank's exchange block instead of memory of its own (tp_common.cuh)
    unsigned char *tp_peer[8];
    const unsigned int *tp_seq;  // device: exchanges completed before this step
    int tp_rank, tp_size, tp_index;  // this exchange is number tp_index of the step
    unsigned long long *trace;  // optional profiling aid (small-M kernel): [CTA][8] global-timer stamps
};

__device__ __forceinline__ uint64_t umma_desc(const void *smem_tile) {
    // K-major, 128-byte swizzle: rows are 128 bytes, 8-row groups are 1024 bytes apart (SBO);
    // descriptor version 1 (sm_100), layout type 2 = SWIZZLE_128B.
    const uint64_t addr = smem_u32(smem_tile);
    return ((addr & 0x3FFFFull) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float silu_gemm(float x) { return __fdiv_rn(x, 1.0f + expf(-x)); }


// [rows][k] FP16 row-major as a 2-D tensor map with a 64 x box_rows box and 128-byte swizzle (gemm_tc.cu).
int make_map(CUtensorMap *map, const void *base, int rows, int k, int box_rows);

// The small-M path of llmb_gemm_f16 (gemm_smallm.cu): m <= 32 rows.
int launch_gemm_smallm(const LlmbGemmArgs *a, cudaStream_t stream);

}  // namespace llmb
