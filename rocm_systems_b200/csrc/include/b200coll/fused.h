/*
 * Fused compute + communication entry points of b200coll (no counterpart in the NCCL API).
 * All of them enqueue on `stream` and return at once; buffers are device pointers.
 */
#ifndef B200COLL_FUSED_H_
#define B200COLL_FUSED_H_

#include "b200coll/nccl.h"

#ifdef __cplusplus
extern "C" {
#endif

/* FSDP gradient bucket: reduce-scatter of bf16 inputs (nranks * recvcount elements per rank)
 * with fp32 accumulation, multiplied by `scale`, written as fp32 (recvcount elements). */
ncclResult_t b200collReduceScatterCast(ncclComm_t comm, const void* sendBf16, float* recvF32, size_t recvcount, float scale,
                                       cudaStream_t stream);

/* Tensor-parallel all-gather -> GEMM in one tcgen05 kernel.
 * xSym: this rank's copy of X [nranks * rowsPerRank, K] bf16 inside symmetric memory, with this
 * rank's shard already at rows [rank * rowsPerRank, +rowsPerRank). The kernel pulls the other
 * shards from the peers while it multiplies: out = X * w^T with w [wRows, K] bf16 (K-major).
 * swiglu != 0: w holds, per block of 256 (or 128) rows, first the gate rows then the up rows of
 * the same outputs, and out [M, wRows / 2] = silu(gate) * up; else out is [M, wRows].
 * commCtas: CTAs that pull the peers' rows (> 0), or 0 = the library's choice: 20 CTAs up to three ranks, copy engines from four
 * ranks up (where they measured 17 % faster). commCtas < 0: no CTA pulls; copy engines do, on a side
 * stream of the library, with stream memory writes publishing the row blocks, and every SM runs the GEMM. In that mode the
 * communicator must not run another collective at the same time (the side stream uses its barrier). */
ncclResult_t b200collAgGemm(ncclComm_t comm, void* xSym, const void* w, void* out, int rowsPerRank, int wRows, int K, int swiglu,
                            int commCtas, cudaStream_t stream);

/* Tensor-parallel GEMM -> reduce-scatter in one tcgen05 kernel.
 * a [nranks * rowsPerRank, K] bf16 and w [N, K] bf16 are this rank's K-shards; y [rowsPerRank, N]
 * bf16 receives rows [rank * rowsPerRank, +rowsPerRank) of sum_over_ranks(a * w^T).
 * workspaceSym: zero-initialised symmetric memory of b200collGemmRsWorkspaceBytes() bytes, the
 * same allocation on every call of a sequence. */
size_t b200collGemmRsWorkspaceBytes(int rowsPerRank, int N, int nranks);
ncclResult_t b200collGemmRs(ncclComm_t comm, const void* a, const void* w, void* workspaceSym, void* y, int rowsPerRank, int N, int K,
                            cudaStream_t stream);

/* The same two kernels on block-scaled fp8 (e4m3) operands. Activations: one fp32 scale per row and 128 channels, stored
 * [K / 128][rows]; weights: one scale per 128 x 128 block, stored [rows / 128][K / 128]. K and the weight rows are
 * multiples of 128; tiles are 128 x 128, and with swiglu != 0 the weight holds, per block of 128 rows, 64 gate rows then
 * the 64 up rows of the same outputs.
 * AgGemmFp8: x8Sym [nranks * rowsPerRank, K] e4m3 and sASym [K / 128][nranks * rowsPerRank] both live in symmetric memory
 * with this rank's rows (and their scales) in place; the kernel pulls rows and scales of the other ranks. out is bf16.
 * GemmRsFp8: a8 / sA and w8 / sW are this rank's K-shards; workspace and y as for b200collGemmRs. A workspace serves
 * either the bf16 or the fp8 form, not both. */
ncclResult_t b200collAgGemmFp8(ncclComm_t comm, void* x8Sym, float* sASym, const void* w8, const float* sW, void* out, int rowsPerRank, int wRows,
                               int K, int swiglu, int commCtas, cudaStream_t stream);
ncclResult_t b200collGemmRsFp8(ncclComm_t comm, const void* a8, const float* sA, const void* w8, const float* sW, void* workspaceSym, void* y,
                               int rowsPerRank, int N, int K, cudaStream_t stream);

/* ---- Mixture-of-experts expert parallelism (experts e*expertsLocal .. on rank e) ----------------
 * One symmetric window of b200collEpWorkspaceBytes() bytes (zero-initialised) per MoE layer holds
 * the per-expert receive buffers (fp8 rows + one fp32 scale per 128 channels), their row counters
 * and the experts' bf16 outputs. `cap` rows are reserved per local expert (multiple of 128); rows
 * beyond it are dropped and counted. hidden: multiple of 1024, at most 7168; k <= 8.
 * A layer runs  Route -> Dispatch -> Experts -> Combine  on one stream. */
size_t b200collEpWorkspaceBytes(int nranks, int expertsLocal, int cap, int hidden, int ffn);
/* top-k expert ids (largest logit first) and softmax-of-selected gate weights per token. */
ncclResult_t b200collEpRoute(const float* logits, int* topIdx, float* topW, int T, int E, int k, cudaStream_t stream);
/* Quantise to fp8 e4m3 and put every (token, expert) row into the owning rank's buffer, from
 * inside one kernel; sentSlot [T, k] receives the row index reserved at the destination (or -1). */
ncclResult_t b200collEpDispatch(ncclComm_t comm, void* winSym, const void* xBf16, const int* topIdx, int* sentSlot, int T, int k,
                                int expertsLocal, int cap, int hidden, int ffn, cudaStream_t stream);
/* Dequantise the received rows and run the two grouped expert GEMMs (SwiGLU between them) on
 * tcgen05. w13 [expertsLocal * 2 ffn, hidden]: per expert, per 256 (128) rows, gate rows then up
 * rows; w2 [expertsLocal * hidden, ffn]. xb / act: scratch [expertsLocal * cap, hidden / ffn] bf16. */
ncclResult_t b200collEpExperts(ncclComm_t comm, void* winSym, const void* w13, const void* w2, void* xb, void* act, int expertsLocal, int cap,
                               int hidden, int ffn, cudaStream_t stream);
/* The same with the first GEMM on the received fp8 rows as they are (no dequantisation pass, no xb): w13Fp8
 * [expertsLocal * 2 ffn, hidden] e4m3 with, per block of 128 rows, 64 gate rows then the 64 up rows of the same outputs,
 * and w13Scales [expertsLocal * 2 ffn / 128][hidden / 128], one fp32 scale per 128 x 128 block. w2 stays bf16. */
ncclResult_t b200collEpExpertsFp8(ncclComm_t comm, void* winSym, const void* w13Fp8, const float* w13Scales, const void* w2, void* act, int expertsLocal,
                                  int cap, int hidden, int ffn, cudaStream_t stream);
/* out [T, hidden] bf16 = sum_k gate[t, k] * expert_output(row sent for (t, k)), pulled from the
 * owning ranks inside one kernel, in the order k = 0 .. k-1. */
ncclResult_t b200collEpCombine(ncclComm_t comm, void* winSym, const int* topIdx, const float* topW, const int* sentSlot, void* out, int T, int k,
                               int expertsLocal, int cap, int hidden, int ffn, cudaStream_t stream);
ncclResult_t b200collEpCounts(ncclComm_t comm, void* winSym, int expertsLocal, int cap, int hidden, int ffn, unsigned int* countsHost,
                              int* droppedHost, cudaStream_t stream);

/* Backward pass of the layer, on the rows and slots of the latest dispatch (nothing is reserved or counted again):
 *   GateGrad     dGate [T, k] fp32 = <dy[t], expert output row of (t, k)>, at the tokens' home rank; run it before any
 *                grouped GEMM writes the window's output region again.
 *   GatherGrad   at the experts' rank: dOut [expertsLocal * cap, hidden] bf16 = gate * dy of each arrived row's token, pulled
 *                from the token's home rank. dySym [T, hidden] bf16 and gateSym [T, k] fp32 are symmetric memory that every
 *                rank filled earlier on its stream; a barrier inside orders them before the pulls.
 *   GroupedGemm  out[rows of e] = a[rows of e] * w[e]^T per local expert (a [expertsLocal * cap, K], w [expertsLocal * wRows, K],
 *                out [expertsLocal * cap, wRows]; nullptr: the window's output region, wRows == hidden), skipping row blocks
 *                without tokens: with transposed weights, the experts' input-gradient GEMMs.
 * The input gradient is then b200collEpCombine with unit weights. */
ncclResult_t b200collEpGateGrad(ncclComm_t comm, void* winSym, const void* dy, const int* topIdx, const int* sentSlot, float* dGate, int T, int k,
                                int expertsLocal, int cap, int hidden, int ffn, cudaStream_t stream);
ncclResult_t b200collEpGatherGrad(ncclComm_t comm, void* winSym, const void* dySym, const void* gateSym, void* dOut, int T, int k, int expertsLocal,
                                  int cap, int hidden, int ffn, cudaStream_t stream);
ncclResult_t b200collEpGroupedGemm(ncclComm_t comm, void* winSym, const void* a, const void* w, void* out, int wRows, int K, int expertsLocal, int cap,
                                   int hidden, int ffn, cudaStream_t stream);

/* ---- RMSNorm backward for callers that may not allocate device memory (no counterpart in the reference) -------------
 * dx [T, H] and dw [H] (both bf16) of y = x * rstd * w; the fp32 accumulator of dw is a fixed 32 KiB array inside the
 * library instead of caller memory, so the call makes no cudaMalloc / cudaFree. H: a multiple of 8, at most 8192 (wider
 * rows are refused with -2 and a message). All calls on a GPU share that array: calls that may overlap on one GPU must
 * be ordered by the caller. The first call on a device resolves the array's address (and may make the driver load this
 * library's kernels): make it outside of stream capture. The full rules are in csrc/fused/no_alloc.h of the source tree. */
int b200ops_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dwBf16, long long T, int H,
                                cudaStream_t stream);
const char* b200ops_rmsnorm_bwd_noalloc_error(void);

#ifdef __cplusplus
}
#endif

#endif /* B200COLL_FUSED_H_ */
