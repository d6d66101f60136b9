/*
 * woq_b200.h -- C ABI of libwoq_b200.so: weight-only-quantised (WOQ) linear for NVIDIA B200
 * (sm_100a).
 *
 * The library replaces the kernel layer of intel-extension-for-pytorch's WOQ linear.  Every
 * entry point names the reference interface it stands in for (paths are relative to the
 * reference project).  All pointers are plain device pointers unless stated otherwise; no
 * framework types cross this boundary.  Calls are asynchronous on the CUDA stream passed in
 * (a `cudaStream_t` carried as `void*`), never throw and never abort: they return one of the
 * WOQ_B200_* status codes, and `woq_b200_last_error()` gives a message for the calling thread.
 *
 * Numeric contract (same as the reference's bf16 / int8 compute modes):
 *   INT4/INT8 weights, lowp BF16:  y = bf16( sum_k x[m,k] * W[n,k] + bias[n] ), then post-op,
 *       W[n,k] = (q[n,k] - zp[n,g]) * bf16(scale[n,g]), fp32 accumulation.
 *   INT8 weights, lowp INT8:       per-token symmetric int8 activations, int32 accumulation,
 *       y = bf16( float(acc) * scale_a[m] * scale_w[n] + bias[n] ), then post-op.
 *   Everything else the reference routes (NF4 / FP8 / INT8 weights with floating compute, fp16
 *   and fp32 compute, shapes off the 64-element grid): woq_b200_linear_any.
 */
#ifndef WOQ_B200_H_
#define WOQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------- */
#define WOQ_B200_OK 0
#define WOQ_B200_ERR_INVALID_ARG 1   /* null pointer, bad size, misaligned buffer          */
#define WOQ_B200_ERR_UNSUPPORTED 2   /* a valid reference configuration this build lacks   */
#define WOQ_B200_ERR_CUDA 3          /* a CUDA runtime call failed                         */
#define WOQ_B200_ERR_WORKSPACE 4     /* workspace smaller than woq_b200_workspace_bytes()  */
#define WOQ_B200_ERR_BAD_HANDLE 5    /* context pointer does not carry the magic word      */
#define WOQ_B200_ERR_DEVICE_WAIT 6   /* a bounded in-kernel wait ran out (status word set) */

/* ---- enumerations shared with the reference (csrc/cpu/aten/utils/woq_defines.h:6-50) -- */
#define WOQ_B200_DTYPE_INT8 1
#define WOQ_B200_DTYPE_INT4 2
#define WOQ_B200_DTYPE_NF4 3
#define WOQ_B200_DTYPE_FP8 4

#define WOQ_B200_LOWP_NONE 0
#define WOQ_B200_LOWP_FP16 1
#define WOQ_B200_LOWP_BF16 2
#define WOQ_B200_LOWP_INT8 3

/* Dynamic activation quantisation of the INT8 compute path (woq_defines.h:11-19): one range
 * for the whole activation tensor, per K block (shared by all tokens), per token, or per token
 * and K block; asymmetric u8 codes with a zero point, or (+4) symmetric s8 codes. */
#define WOQ_B200_ACT_NONE (-1)
#define WOQ_B200_ACT_PER_TENSOR 0
#define WOQ_B200_ACT_PER_K_BLOCK 1
#define WOQ_B200_ACT_PER_M 2
#define WOQ_B200_ACT_PER_M_K_BLOCK 3
#define WOQ_B200_ACT_PER_TENSOR_SYM 4
#define WOQ_B200_ACT_PER_K_BLOCK_SYM 5
#define WOQ_B200_ACT_PER_M_SYM 6
#define WOQ_B200_ACT_PER_M_K_BLOCK_SYM 7

#define WOQ_B200_FMT_PLAIN 0 /* INT4: [N, K/2] u8, even k in the low nibble; INT8: [N, K] s8 */
#define WOQ_B200_FMT_GPTQ 1  /* [K/8, N] int32                                             */
#define WOQ_B200_FMT_AWQ 2   /* [K, N/8] int32, nibble order 0,2,4,6,1,3,5,7               */

/* post-op codes (woq_defines.h:27-38) */
#define WOQ_B200_FUSE_NONE 0x0
#define WOQ_B200_FUSE_GELU_ERF 0x1
#define WOQ_B200_FUSE_GELU_TANH 0x2
#define WOQ_B200_FUSE_RELU 0x3
#define WOQ_B200_FUSE_SILU 0x4
#define WOQ_B200_FUSE_ADD 0x10
#define WOQ_B200_FUSE_ADD_ADD 0x20
#define WOQ_B200_FUSE_MUL 0x30
/* Not in the reference: y[M,N/2] = bf16(up * silu(gate)) for a weight that stacks gate rows
 * [0,N/2) over up rows [N/2,N).  Equals woq_linear_silu followed by woq_linear_mul
 * (intel_extension_for_pytorch/transformers/models/cpu/fusions/linear_fusion.py:482-490).
 * Needs a context created with WOQ_B200_LAYOUT_GATE_UP. */
#define WOQ_B200_FUSE_SILU_MUL 0x100
/* Not in the reference as a post-op: out[row_idx[i], :] = bf16(out + y[i,:] * row_w[i]), the
 * scatter step of mixtral_moe_woq (csrc/cpu/aten/kernels/MoEKrnl.cpp:67-120). */
#define WOQ_B200_FUSE_SCALED_SCATTER_ADD 0x200

/* element types of the tensors handed to woq_b200_ctx_create */
#define WOQ_B200_T_NONE 0
#define WOQ_B200_T_F32 1
#define WOQ_B200_T_F16 2
#define WOQ_B200_T_BF16 3
#define WOQ_B200_T_U8 4
#define WOQ_B200_T_S8 5
#define WOQ_B200_T_I32 6 /* packed 4-bit zero points of GPTQ/AWQ checkpoints */

#define WOQ_B200_LAYOUT_GATE_UP 0x1
/* An INT4 context normally keeps the weight in two tilings (streaming kernel / tensor-core
 * kernel).  These flags keep only one, halving device memory; calls then always use the
 * kernel whose tiling exists (the streaming kernel takes large M in 16-token passes). */
#define WOQ_B200_LAYOUT_STREAM_ONLY 0x2
#define WOQ_B200_LAYOUT_TC_ONLY 0x4
/* GPTQ / AWQ weights whose scales and zero points were already brought to [N, groups]
 * (what the reference's Python loaders hand to weight_only_qlinear_prepack_int4). */
#define WOQ_B200_LAYOUT_SCALES_NK 0x8
/* woq_b200_ctx_create validates the zero points on the device.  Normally it waits for the
 * outcome (one stream synchronisation per context); with this flag the outcome travels to the
 * host asynchronously and the first woq_b200_linear* call on the context reports it, so a
 * loader can create hundreds of contexts back to back.  The inputs must stay alive until the
 * stream has passed the create call either way.  Plain-format INT4 contexts only. */
#define WOQ_B200_LAYOUT_DEFER_CHECK 0x10
/* Keep the weight in its plain layout and run it through the general kernel (any weight dtype,
 * fp32 / fp16 / bf16 compute, any K, group sizes that are multiples of 8).  Descriptions the
 * tuned kernels do not take (NF4 / FP8 weights, INT8 weights without INT8 compute, lowp FP16,
 * K not a multiple of 64, group sizes below 64) get this route without the flag; set it to run
 * an INT4 layer on fp32 or fp16 activations under lowp NONE. */
#define WOQ_B200_LAYOUT_GENERIC 0x20

/* kernel selection for INT4 weights.  AUTO, TENSOR_CORE and STREAM all multiply by the
 * bf16-rounded dequantised weights bf16((q - zp) * bf16(scale)) and differ only in summation
 * order.  STREAM_FAST applies scale and zero point after the sum over each 64-wide k-block
 * (what the reference's small-M kernel does after each group,
 * csrc/cpu/aten/utils/woq.h:784-951): about 10 % faster on large layers, exact on one-hot
 * inputs, and for a single linear within the output tolerance (mean relative deviation
 * 1.2e-3 .. 1.7e-3 from the per-weight form on every benchmark shape, bar 2e-3) - but not the
 * same rounding as the tile dequantiser, and a product of two such linears (the gate/up
 * epilogue, woq_linear_silu followed by woq_linear_mul) deviates by about 2.5e-3, over the
 * bar; so it is never chosen automatically.  It expects |x| < 2^40 (larger activations
 * overflow to infinity inside the kernel) and treats |x| < 2^-61 as zero. */
#define WOQ_B200_HINT_AUTO 0        /* streaming kernel for M <= 16, tcgen05 kernel above      */
#define WOQ_B200_HINT_TENSOR_CORE 1 /* tcgen05 kernel for every M                              */
#define WOQ_B200_HINT_STREAM 2      /* register-dequant streaming kernel, 16 tokens a pass     */
#define WOQ_B200_HINT_STREAM_FAST 3 /* streaming kernel, scale applied after the k-block sum   */

/* Description of one quantised linear layer: the arguments of
 * ipex_prepack::weight_only_qlinear_prepack
 * (csrc/cpu/jit/cpu/kernels/RegisterOpContextClass.cpp:192-205). */
typedef struct woq_b200_desc {
  int64_t n;              /* out features                                                   */
  int64_t k;              /* in features                                                    */
  int32_t weight_dtype;   /* WOQ_B200_DTYPE_*                                               */
  int32_t group_size;     /* > 0, or -1 for one group per output channel                   */
  int32_t lowp_mode;      /* WOQ_B200_LOWP_*                                                */
  int32_t act_quant_mode; /* WOQ_B200_ACT_*; only read when lowp_mode is INT8               */
  int32_t weight_format;  /* WOQ_B200_FMT_*                                                 */
  int32_t scale_dtype;    /* F32, F16 or BF16; scales are [N, ceil(K/G)] ([K/G, N] for AWQ/GPTQ) */
  int32_t zp_dtype;       /* NONE (symmetric: 8 for INT4, 0 for INT8), F32, U8, or packed
                             int32 words (same packing as the weight) for GPTQ/AWQ         */
  int32_t bias_dtype;     /* NONE, F32 or BF16; bias is [N]                                 */
  int32_t layout_flags;   /* WOQ_B200_LAYOUT_*                                              */
  int32_t kernel_hint;    /* WOQ_B200_HINT_*: 0 lets the library choose per call              */
} woq_b200_desc;

typedef struct woq_b200_ctx woq_b200_ctx; /* opaque; host memory owning device buffers */

/* Library version (major*10000 + minor*100 + patch). No reference counterpart. */
int woq_b200_version(void);

/* Message for the last non-OK status returned to the calling host thread. */
const char* woq_b200_last_error(void);

/* Number of kernels this library has launched in this process (all threads). */
int64_t woq_b200_kernel_launches(void);

/* Process-wide tuning switches.  No reference counterpart (the reference reads its tuning from
 * environment variables, e.g. csrc/cpu/aten/utils/woq.h block-size getters).  Set them while no
 * call of this library is in flight on another host thread.
 *   WOQ_B200_OPT_DECODE_SPLIT: how the M <= 16 INT4 kernel cuts a layer whose K range is
 *     shared by several thread blocks.  0 (default, or WOQ_B200_DECODE_SPLIT in the
 *     environment at load time): chosen per layer; 1: always the stream-K grid that reduces
 *     split tiles through the workspace; 2: thread-block clusters that reduce through
 *     distributed shared memory whenever the layer has at most two tiles per SM. */
#define WOQ_B200_OPT_DECODE_SPLIT 1
int woq_b200_set_option(int32_t option, int32_t value);

/* Repack a plain quantised weight into the tiled device layout and keep bf16 scales,
 * zero points and fp32 bias beside it.  Replaces woq_linear_pack_weight + qlinear_woq_pack
 * (csrc/cpu/aten/Linear.cpp:379-438, csrc/cpu/aten/kernels/WoqUtilKrnl.cpp:32-249) and the
 * scale/zero-point re-layout of ContextLinearWoq (csrc/cpu/jit/cpu/kernels/ContextLinearWoq.h:36-128).
 * Allocates the packed buffers with cudaMalloc on the current device; inputs may be freed
 * once the stream has passed this call.  Synchronises the stream once to validate the zero
 * points (see WOQ_B200_LAYOUT_DEFER_CHECK). */
int woq_b200_ctx_create(const woq_b200_desc* desc, const void* qweight, const void* scales,
                        const void* zero_points, const void* bias, void* stream,
                        woq_b200_ctx** out);

/* Frees the packed buffers.  Counterpart of the op-context destructor
 * (csrc/cpu/jit/cpu/kernels/OpContext.h:363-405). */
int woq_b200_ctx_destroy(woq_b200_ctx* ctx);

/* Copy of the descriptor a context was created with. */
int woq_b200_ctx_desc(const woq_b200_ctx* ctx, woq_b200_desc* out);

/* Which kernels a context runs on (decided by woq_b200_ctx_create from the description):
 * the tuned INT4 / bf16 kernels, the tcgen05 INT8 kernel (INT8 weights, whole-K activation
 * ranges), the general kernel (woq_b200_linear_any), or the K-block INT8 kernel.  -1: not a
 * context.  No reference counterpart (the reference picks its kernel per call,
 * csrc/cpu/aten/kernels/WoqLinearKrnl.cpp:56-165). */
#define WOQ_B200_ROUTE_INT4_BF16 0
#define WOQ_B200_ROUTE_INT8 1
#define WOQ_B200_ROUTE_GENERAL 2
#define WOQ_B200_ROUTE_INT8_BLOCK 3
int woq_b200_ctx_route(const woq_b200_ctx* ctx);

/* Bytes of the packed weight + scale buffers held on the device. */
size_t woq_b200_ctx_device_bytes(const woq_b200_ctx* ctx);

/* Bit-exact inverse of the repack: writes the plain [N, K/2] u8 (INT4) or [N, K] s8 (INT8)
 * weight.  Replaces qlinear_woq_unpack (csrc/cpu/aten/kernels/WoqUtilKrnl.cpp:251-324). */
int woq_b200_ctx_unpack(const woq_b200_ctx* ctx, void* qweight_plain, void* stream);

/* Scratch bytes woq_b200_linear needs for M tokens.  The first woq_b200_workspace_header_bytes()
 * bytes must be zero before the first use of a workspace (cudaMemsetAsync once); every call
 * leaves them zero again, so one workspace can be reused by any number of stream-ordered
 * calls.  Calls that overlap on the device need separate workspaces. */
size_t woq_b200_workspace_bytes(const woq_b200_ctx* ctx, int64_t m);
size_t woq_b200_workspace_header_bytes(void);

/* y[M, N_out] (bf16) = post_op( x[M, K] (bf16) * W^T + bias ).  Replaces the kernel reached
 * from torch_ipex::ipex_woq_linear / woq_linear_{gelu,new_gelu,relu,silu,add,add_add,mul}
 * (csrc/cpu/aten/Linear.cpp:499-811 -> qlinear_woq_affine,
 * csrc/cpu/aten/kernels/WoqLinearKrnl.cpp:56-165).  `others` is a HOST array of n_others
 * device pointers to [M, N] bf16 tensors (ADD: 1, ADD_ADD: 2, MUL: 1).  x rows are ldx
 * elements apart; y rows AND the rows of the extra tensors are ldy elements apart (pass K and
 * N_out for dense tensors).  N_out = N, or N/2 for WOQ_B200_FUSE_SILU_MUL.  The current device
 * must be the one the context was created on. */
int woq_b200_linear(const woq_b200_ctx* ctx, const void* x, int64_t m, int64_t ldx, int32_t fusion,
                    const void* const* others, int32_t n_others, void* y, int64_t ldy,
                    void* workspace, size_t workspace_bytes, void* stream);

/* woq_b200_linear for activations, outputs and extra tensors of `io_dtype` (WOQ_B200_T_BF16,
 * _F16 or _F32).  The compute dtype follows the reference's routing
 * (csrc/cpu/aten/kernels/WoqLinearKrnl.cpp:75-165): lowp BF16 -> bf16, lowp FP16 -> fp16, lowp
 * NONE -> the activation's dtype; W = round_c((code - zp) * round_c(scale)) with round_c the
 * rounding to the compute dtype (none for fp32), activations rounded to it, fp32 accumulation,
 * result rounded to io_dtype, post-op on io_dtype data.  Codes: INT4 0..15, NF4 through the
 * reference's table (csrc/cpu/aten/utils/woq_utils.h:34-51), INT8 -128..127, FP8 e4m3 through
 * the reference's conversion (csrc/cpu/aten/utils/woq.h:465-483).  Contexts on the general
 * route take every io_dtype; the others take bf16 only (and forward to woq_b200_linear).
 * No fused silu*mul on the general route. */
int woq_b200_linear_any(const woq_b200_ctx* ctx, const void* x, int32_t io_dtype, int64_t m, int64_t ldx,
                        int32_t fusion, const void* const* others, int32_t n_others, void* y, int64_t ldy,
                        void* workspace, size_t workspace_bytes, void* stream);

/* ---- Tensor-parallel layers on the GPUs of one node ------------------------------------------
 * The reference shards column-parallel layers along N and row-parallel layers along K and
 * exchanges through its communication back end after the linear
 * (intel_extension_for_pytorch/nn/modules/weight_only_quantization.py:536-633,
 * csrc/cpu/aten/kernels/TPPSHMAllreduceAddKrnl.cpp:183-197 for the shared-memory all-reduce).
 * Here the exchange is part of the decode kernel's epilogue: every rank owns a buffer of the
 * same layout ("comm"), maps its peers' buffers through CUDA IPC, and the kernel stores its
 * tile of the result straight into every rank's buffer over NVLink.  All ranks must issue the
 * same sequence of calls on a comm, within about two seconds of each other (a kernel that has
 * waited that long for a peer gives up and sets the workspace status).  One process per GPU; at most 8 ranks; 1..16 tokens. */
typedef struct woq_b200_comm woq_b200_comm;
#define WOQ_B200_COMM_HANDLE_BYTES 64

/* Allocates this rank's buffer on the current device: exchange slots for layers whose local
 * weight has up to max_n rows (row-parallel: N; column-parallel: this rank's N shard) and a
 * gather area of gather_bytes. */
int woq_b200_comm_create(int32_t rank, int32_t world, int64_t max_n, size_t gather_bytes,
                         woq_b200_comm** out);
/* Writes the 64-byte handle the other ranks need to map this rank's buffer. */
int woq_b200_comm_export(const woq_b200_comm* comm, void* handle);
/* `handles`: world x 64 bytes in rank order (this rank's own entry is ignored). */
int woq_b200_comm_connect(woq_b200_comm* comm, const void* handles);
/* Device address of this rank's gather area. */
void* woq_b200_comm_gather_ptr(const woq_b200_comm* comm);
int woq_b200_comm_destroy(woq_b200_comm* comm);

/* Row-parallel linear fused with the all-reduce: x[M, K_local], this rank's K shard of the
 * weight; y[M, N] = post_op( bf16(sum over ranks of bf16(x_r W_r^T)) + bias ) on every rank,
 * the partial outputs added in rank order in fp32 (IpexWoqLinearAllreduce.forward ->
 * all_reduce_and_bias_add, nn/utils/_weight_prepack.py:139-158).  `bias`: fp32 [N] on the
 * device or null; the context itself must have been packed without bias. */
int woq_b200_linear_allreduce(const woq_b200_ctx* ctx, const woq_b200_comm* comm, const void* x,
                              int64_t m, int64_t ldx, int32_t fusion, const void* const* others,
                              int32_t n_others, const float* bias, void* y, int64_t ldy,
                              void* workspace, size_t workspace_bytes, void* stream);

/* Column-parallel linear fused with the all-gather: this rank's N shard; the gathered
 * [M, world * N_out_local] bf16 tensor appears at byte `gather_offset` of every rank's
 * gather area (rank r's columns at r * N_out_local).  This rank's own column block is there
 * when the kernel has finished; the other ranks' blocks arrive over NVLink without anybody
 * waiting for them and are put in place by the NEXT fused call on the same comm (while its
 * weights stream) or by woq_b200_comm_fence: the whole tensor is complete when that call has
 * finished.  A consumer that only reads its own block (a row-parallel layer behind a
 * column-parallel one, as in the reference's tensor-parallel chain,
 * intel_extension_for_pytorch/nn/modules/weight_only_quantization.py:536-633) never waits.
 * A gather destination may be written again only after a later exchange on the same comm has
 * completed on this rank.  A sequence of fused calls captured in a CUDA graph must begin and
 * end with no gather outstanding (call woq_b200_comm_fence before the capture, and let a
 * reduce or a fence be the last captured call). */
int woq_b200_linear_allgather(const woq_b200_ctx* ctx, const woq_b200_comm* comm, const void* x,
                              int64_t m, int64_t ldx, int32_t fusion, const void* const* others,
                              int32_t n_others, size_t gather_offset, void* workspace,
                              size_t workspace_bytes, void* stream);

/* Completes an outstanding all-gather on this rank without running a linear (a small kernel
 * on `stream` that waits, bounded, for the other ranks' column blocks and puts them in place).
 * No-op when nothing is outstanding.  woq_b200_comm_status then reports, after synchronising the
 * stream, whether that kernel gave up waiting (WOQ_B200_ERR_DEVICE_WAIT). */
int woq_b200_comm_fence(woq_b200_comm* comm, void* stream);
int woq_b200_comm_status(woq_b200_comm* comm, void* stream);

/* No counterpart in the reference.  Same computation as woq_b200_linear for at most 16 tokens,
 * for callers that may not allocate device memory (memory-planned graphs, servers that forbid
 * allocation after start-up, sandboxes without a re-entrant allocator): the scratch lives in a
 * 4 MiB array inside the library's device image, held by every GPU that loads the library
 * until the process exits.  Calls no cudaMalloc / cudaFree.  Returns WOQ_B200_ERR_INVALID_ARG
 * for m > 16 and WOQ_B200_ERR_WORKSPACE when the GPU would need more than the 4 MiB (more than
 * 252 SMs).  The first call on each device looks up the array's address; make that call
 * outside any stream capture.  All calls on one GPU share the array: they must be
 * stream-ordered, two that overlap on the device race on the partial tiles and counters.  The
 * current device must be the one the context was created on (the array used is the current
 * device's). */
int woq_b200_linear_static_scratch(const woq_b200_ctx* ctx, const void* x, int64_t m, int64_t ldx,
                                   int32_t fusion, const void* const* others, int32_t n_others,
                                   void* y, int64_t ldy, void* stream);

/* No counterpart in the reference.  woq_b200_workspace_status for the built-in array of the
 * current device: synchronises the stream, returns WOQ_B200_ERR_DEVICE_WAIT if a kernel of an
 * earlier woq_b200_linear_static_scratch call gave up a bounded wait (its output is then not
 * valid), and clears the record.  Until it is called the record stays, and later kernels on the
 * array do not wait either. */
int woq_b200_static_scratch_status(void* stream);

/* One expert of a mixture-of-experts layer on gathered tokens:
 * out[row_idx[i], :] = bf16(out[row_idx[i], :] + y[i, :] * row_weight[i]) with
 * y = x[row_idx_in ? row_idx_in[i] : i, :] * W^T.  Replaces fuse_index_unsqueeze /
 * fuse_index_mul_index_add around the WOQ linears of mixtral_moe_woq
 * (csrc/cpu/aten/kernels/MoEKrnl.cpp:67-160,254-285).  row_weight is bf16 [m].  The row_idx
 * values of one call must be distinct (a token reaches an expert once); rows that repeat
 * would lose all but one of their updates. */
int woq_b200_linear_scatter(const woq_b200_ctx* ctx, const void* x, int64_t m, int64_t ldx,
                            const int32_t* row_idx, const void* row_weight, void* out,
                            int64_t ld_out, void* workspace, size_t workspace_bytes,
                            void* stream);

/* One expert of a Mixtral-style layer in one call: gather the expert's tokens
 * x = hidden[token_idx[i], :], a = silu(gate(x)) * up(x) on the stacked gate/up weight `w13`
 * (created with WOQ_B200_LAYOUT_GATE_UP), y = w2(a), out[token_idx[i], :] = bf16(out + y[i] * w[i]).
 * Replaces mixtral_moe_woq_kernl_impl (csrc/cpu/aten/kernels/MoEKrnl.cpp:254-285).  token_weight is
 * bf16 [tokens]; a token may appear at most once per call. */
size_t woq_b200_moe_workspace_bytes(const woq_b200_ctx* w13, const woq_b200_ctx* w2, int64_t tokens);
int woq_b200_moe_expert(const woq_b200_ctx* w13, const woq_b200_ctx* w2, const void* hidden, int64_t ldh,
                        const int32_t* token_idx, const void* token_weight, int64_t tokens, void* out,
                        int64_t ld_out, void* workspace, size_t workspace_bytes, void* stream);

/* RMSNorm fused with the per-token activation quantiser of the INT8 path.  For every row of
 * x (bf16 [m, k], k a multiple of 16):
 *   y  = bf16(x * rsqrt(mean(x^2) + eps) * gamma)        fp32 arithmetic, one rounding; gamma bf16 [k]
 *   qa = the int8 codes of y, sa its scale, zpa its zero point (asymmetric mode only), computed as
 *        woq_b200_linear computes them for a context with the same act_quant_mode
 *        (dynamic_quantize_per_block, csrc/cpu/aten/utils/woq_dynamic_quant.h:1526-1750)
 * so that several linears which read the same normalised activations (q/k/v, gate/up) share one
 * quantisation and y never makes a round trip through memory.  y may be null.
 * act_quant_mode: WOQ_B200_ACT_PER_M or WOQ_B200_ACT_PER_M_SYM.  qa is [m, k] bytes (row stride k),
 * sa [m] floats, zpa [m] int32.  This is a B200-side fusion: the reference runs the norm and the
 * quantiser as separate steps (it has no fused form). */
int woq_b200_rmsnorm_quant(const void* x, int64_t ldx, const void* gamma, float eps, int64_t m, int64_t k,
                           int32_t act_quant_mode, void* y, int64_t ldy, void* qa, void* sa, void* zpa,
                           void* stream);

/* woq_b200_linear on activations that are already quantised (by woq_b200_rmsnorm_quant, or taken
 * from woq_b200_int8_internals): codes qa [m, K], scales sa [m], zero points zpa [m] (null for the
 * symmetric mode).  The context must be on the tcgen05 INT8 route (INT8 weights, lowp INT8) with a
 * per-token act_quant_mode, and the codes must have been made in that mode.  Everything else
 * (fusion, others, y, workspace of woq_b200_workspace_bytes(ctx, m) bytes) as in woq_b200_linear. */
int woq_b200_linear_prequant(const woq_b200_ctx* ctx, const void* qa, const void* sa, const void* zpa, int64_t m,
                             int32_t fusion, const void* const* others, int32_t n_others, void* y, int64_t ldy,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Parity hooks -------------------------------------------------------------------------
 * Dequantised weight [N, K] bf16 produced by the same device routine the tensor-core kernel
 * uses for its tiles (the reference's Dequantize<bfloat16>, csrc/cpu/aten/utils/woq.h:1501-1581). */
int woq_b200_dump_dequant(const woq_b200_ctx* ctx, void* w_bf16, void* stream);

/* The same for a general-route context: [N, K] fp32 holding the values the kernel multiplies by
 * when it computes in `compute_dtype` (WOQ_B200_T_BF16 / _F16 / _F32). */
int woq_b200_dump_dequant_f32(const woq_b200_ctx* ctx, int32_t compute_dtype, float* w_f32, void* stream);

/* INT8-lowp internals for M tokens: quantised activations qa[M, K] (s8, or u8 in the
 * asymmetric modes), their scales sa[M] f32 (dynamic_quantize_per_block,
 * csrc/cpu/aten/utils/woq_dynamic_quant.h:1526-1750) and the int32 accumulators acc[M, N]
 * = sum over the whole K of qa * qw, before the zero-point compensation (woq.h:2231-2354).
 * Any of the three outputs may be null. */
int woq_b200_int8_internals(const woq_b200_ctx* ctx, const void* x, int64_t m, int64_t ldx,
                            int8_t* qa, float* sa, int32_t* acc, void* workspace,
                            size_t workspace_bytes, void* stream);

/* The same for the K-block INT8 route (INT4 weights with INT8 compute, grouped INT8 weights, or
 * an activation range per K block: act_quant_mode 1, 3, 5, 7): the activation codes qa[M, K] in
 * natural order (u8 for the asymmetric modes, s8 bit patterns for the symmetric ones), scales
 * sa[M, K / block] and zero points zpa[M, K / block] per token and K block (modes that share a
 * range repeat it), and the int32 block accumulators acc[K / block, M, N] after the weight zero
 * point and the activation compensation (csrc/cpu/aten/utils/woq.h:962-1126).  Any output may
 * be null.  woq_b200_int8_block_size gives the K block (0 for other contexts). */
int woq_b200_int8_block_internals(const woq_b200_ctx* ctx, const void* x, int64_t m, int64_t ldx, uint8_t* qa,
                                  float* sa, int32_t* zpa, int32_t* acc, void* workspace,
                                  size_t workspace_bytes, void* stream);
int woq_b200_int8_block_size(const woq_b200_ctx* ctx);

/* The activation zero points zp[M] (int32) that the latest INT8 call on `workspace` with M
 * tokens left there; zeros for the symmetric modes. */
int woq_b200_int8_zero_points(const woq_b200_ctx* ctx, int64_t m, int32_t* zp, const void* workspace,
                              size_t workspace_bytes, void* stream);

/* How woq_b200_linear would launch the M <= 16 INT4 kernel for this context on the current
 * device (no reference counterpart; a diagnostic): out[0] thread blocks, out[1] thread blocks
 * per cluster (0: the stream-K grid), out[2] k-blocks per warp and pipeline stage, out[3] the
 * shared-memory budget per thread block in bytes. */
int woq_b200_decode_plan(const woq_b200_ctx* ctx, int64_t m, int32_t* out);

/* The pipeline shape of one launch of the tcgen05 INT4 kernel with n_tok token columns (16..256,
 * a multiple of 16; woq_b200_linear rounds the tokens of a launch up to that).  No reference
 * counterpart; a diagnostic that needs no GPU: out[0] k-blocks per stage, out[1] slots of the
 * A-group / activation ring (at least 4), out[2] slots of the packed-weight ring (a multiple of 4),
 * out[3] first TMEM column of the A groups (out[3] + 32 * out[0] * out[1] <= 512), out[4] dynamic
 * shared memory in bytes. */
int woq_b200_tc_plan(int32_t n_tok, int32_t* out);

/* Reads the status word of a workspace (synchronises the stream).  WOQ_B200_OK, or
 * WOQ_B200_ERR_DEVICE_WAIT when a bounded wait inside a kernel gave up; the word is cleared. */
int woq_b200_workspace_status(void* workspace, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WOQ_B200_H_ */
