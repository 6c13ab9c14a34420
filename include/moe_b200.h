/*
 * moe_b200.h -- C ABI of the B200 (sm_100a) MoE feed-forward block for the
 * gpt-oss-amd engine.
 *
 * The library replaces, inside the engine's forward(), the per-layer MoE block
 * of src/forward.cpp:317-992 (router GEMM + bias, top-k, softmax over the
 * selected logits, token->expert permutation, grouped gate/up GEMM with the
 * clamped SwiGLU, grouped down GEMM, routing-weighted combine, and the
 * expert-parallel exchange) and the expert part of the weight loader
 * (src/model.cpp:104-114,365-399).  Expert weights are handed over and kept as
 * packed MXFP4 (32-element e2m1 blocks + e8m0 scales); they are unpacked inside
 * the GEMM kernels.  There is no CPU fallback: every entry point that computes
 * needs a CUDA device of compute capability 10.0.
 *
 * Conventions
 *   - plain C, no exceptions, nothing calls exit(): every function returns a
 *     moe_b200_status (0 = success); moe_b200_last_error() gives the text.
 *     (The reference's CHECK_HIP prints and exits, include/model.hpp:8-17.)
 *   - one handle per GPU, used by one host thread at a time.
 *   - moe_b200_forward() is asynchronous on the caller's stream.  With
 *     ep_size == 1 it never synchronises with the host; with ep_size > 1 it
 *     waits once per call for the per-rank row counts (the sizes of the
 *     all-to-all), as the reference waits for its expert offsets every layer
 *     (src/forward.cpp:340-345,381).
 *   - all sizes are in elements unless a name says bytes.
 */
#ifndef MOE_B200_H
#define MOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct moe_b200_handle_s* moe_b200_handle;
/* ABI-identical to cudaStream_t / CUstream. */
typedef struct CUstream_st* moe_b200_stream;

typedef enum {
    MOE_B200_OK = 0,
    MOE_B200_ERR_INVALID = 1,     /* bad argument or configuration            */
    MOE_B200_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed        */
    MOE_B200_ERR_NO_DEVICE = 3,   /* no sm_100 device (there is no fallback)  */
    MOE_B200_ERR_NOT_LOADED = 4,  /* weights of the layer were not set        */
    MOE_B200_ERR_DEVICE = 5,      /* a kernel reported a bounded wait ran out */
    MOE_B200_ERR_NCCL = 6,        /* an NCCL call failed                      */
    MOE_B200_ERR_UNSUPPORTED = 7  /* valid input outside what is implemented  */
} moe_b200_status;

/* Activation element types accepted by moe_b200_forward(). */
#define MOE_B200_DTYPE_F32 0  /* the engine's s->t buffer (include/model.hpp:113) */
#define MOE_B200_DTYPE_BF16 1 /* already-rounded activations                      */

/* The expert GEMMs are tcgen05 kernels (CTA pairs for large batches, token rows
 * on the accumulator lanes for small ones); moe_b200_config.gemm_impl must be
 * MOE_B200_GEMM_TCGEN05 (= 0). */
#define MOE_B200_GEMM_TCGEN05 0
#ifdef MOE_B200_TEST_AIDS
/* Test-aids build of the library only (compiled with -DMOE_B200_TEST_AIDS, never
 * shipped): a plain warp-MMA kernel with the same inputs, layout and rounding
 * points, used by the parity tests to cross-check the tcgen05 kernels on the
 * device at sizes the CPU oracle cannot reach. */
#define MOE_B200_GEMM_MMA_SYNC 1
#endif

/* Mirrors the MoE-related fields of OssConfig (include/model.hpp:25-48) plus
 * the expert-parallel placement of OssTransformerHybrid (include/model.hpp:
 * 232-237). */
typedef struct {
    int hidden_dim;        /* H, multiple of 64                                */
    int intermediate_dim;  /* I, multiple of 64                                */
    int n_experts;         /* E, global, <= 256                                */
    int experts_per_token; /* K, <= 8                                          */
    int n_layers;          /* layers held by this handle                       */
    float swiglu_alpha;    /* 1.702 in the reference (src/run.cpp:673)         */
    float swiglu_limit;    /* OssConfig.swiglu_limit                           */
    int max_tokens;        /* OssConfig.batch_size: most tokens per call, per rank;
                              with ep_size > 1 the same value on every rank      */
    int ep_rank;           /* this GPU's shard, 0 <= ep_rank < ep_size         */
    int ep_size;           /* 1 = all experts local                            */
    int device;            /* CUDA device ordinal                              */
    int gemm_impl;         /* MOE_B200_GEMM_TCGEN05                            */
} moe_b200_config;

/* Contiguous expert shard of a rank, remainder to the low ranks: the rule of
 * copy_transformer_to_device (src/model.cpp:104-114).  Pure host arithmetic. */
void moe_b200_shard_range(int n_experts, int ep_size, int ep_rank, int* first_expert,
                          int* n_local);

/* Create / destroy.  Replaces the MoE part of copy_transformer_to_device /
 * free_transformer_on_device (src/model.cpp:59,500) and the scratch allocation
 * of src/model.cpp:334-354: the handle owns the packed weights of its shard and
 * a workspace sized for max_tokens; nothing is allocated afterwards. */
moe_b200_status moe_b200_create(const moe_b200_config* cfg, moe_b200_handle* out);
moe_b200_status moe_b200_destroy(moe_b200_handle h);

/* Router weights of one layer: w bf16 [E, H] row-major (the layout
 * gemm_router indexes, src/hip/gemms/gemm_router.hip:91-109), bias fp32 [E].
 * Host or device pointers.  Replaces the router part of src/model.cpp:365-399. */
moe_b200_status moe_b200_set_router(moe_b200_handle h, int layer, const void* w_bf16,
                                    const float* bias);

/* Packed MXFP4 experts of one layer, in checkpoint layout (the input of
 * dequantize_fp4, tools/model_export/gpt-oss-20b/export_model_bin.py:95-133):
 *   blocks1 u8 [n, 2I, H/32, 16]  scales1 u8 [n, 2I, H/32]  bias1 f32 [n, 2I]
 *   blocks2 u8 [n, H,  I/32, 16]  scales2 u8 [n, H,  I/32]  bias2 f32 [n, H]
 * rows of mlp1 gate/up interleaved (src/run.cpp:667-670).  `first_expert` is a
 * GLOBAL expert index; the n experts must lie inside this rank's shard.  Host
 * or device pointers.  The library re-tiles the bytes for its kernels; the
 * values they decode to are unchanged.  Every e8m0 scale byte is accepted, as by
 * dequantize_fp4 (export_model_bin.py:125-129); the one limit: inside ONE weight
 * row the scale bytes of the blocks that hold a non-zero code may span at most
 * 128 binades (the row is kept with an exponent shift that the GEMM applies to
 * its fp32 accumulator).  A row outside that is rejected with
 * MOE_B200_ERR_UNSUPPORTED and the experts of the call stay unset.
 * Replaces the expert part of src/model.cpp:141-186,365-399. */
moe_b200_status moe_b200_set_experts_mxfp4(moe_b200_handle h, int layer, int first_expert, int n,
                                           const uint8_t* blocks1, const uint8_t* scales1,
                                           const float* bias1, const uint8_t* blocks2,
                                           const uint8_t* scales2, const float* bias2);

/* Packed expert file: the experts and routers of a model as the checkpoint has
 * them (e2m1 blocks + e8m0 scales + fp32 biases, expert-major, one page-aligned
 * record per (layer, expert)), written by gpt-oss-amd_b200/expert_file.py.
 * Replaces, for the MoE weights, the fp32 .bin of
 * tools/model_export/gpt-oss-20b/export_model_bin.py:95-133 and the loader's
 * fp32 -> bf16 streaming conversion (src/model.cpp:8-56,141-186); everything
 * else stays in the engine's .bin (src/run.cpp:196-235).
 * moe_b200_expert_file_info reads and validates the header (pure host code; any
 * output pointer may be NULL).  moe_b200_load_experts_file maps the file and
 * uploads layer `file_layer` of it into layer `layer` of the handle: the router
 * and the records of THIS rank's expert shard only -- other ranks' records are
 * never touched.  The file's hidden_dim, intermediate_dim, n_experts and
 * experts_per_token must equal the handle's. */
moe_b200_status moe_b200_expert_file_info(const char* path, int* n_layers, int* n_experts,
                                          int* hidden_dim, int* intermediate_dim,
                                          int* experts_per_token, float* swiglu_limit,
                                          unsigned long long* file_bytes);
moe_b200_status moe_b200_load_experts_file(moe_b200_handle h, const char* path, int file_layer,
                                           int layer);

/* The MoE block of one layer for n_tokens rows (src/forward.cpp:317-514, and
 * :515-992 when ep_size > 1).
 *   t            device, [n_tokens, H], f32 or bf16 (f32 is rounded to bf16 on
 *                load, as src/hip/BLAS.hip:32-40 does)
 *   out          device f32 [n_tokens, H]; accumulate == 0: out = e_agg;
 *                accumulate != 0: out += e_agg (the residual add of
 *                src/hip/vecadd.hip:19-38 fused into the combine)
 *   router_score_out / topk_i_out / topk_w_out   optional device buffers
 *                [n_tokens, E] f32 / [n_tokens, K] i32 / [n_tokens, K] f32: the
 *                engine's observable side buffers (include/model.hpp:132-134);
 *                topk_w is after the softmax
 * `t` and `out` must be 16-byte aligned (rows are moved 16 bytes at a time); a
 * pointer that is not is refused with MOE_B200_ERR_INVALID.
 * With ep_size > 1 every rank must call this for the same layer in the same
 * order (n_tokens may differ per rank, 0 included). */
moe_b200_status moe_b200_forward(moe_b200_handle h, int layer, const void* t, int t_dtype,
                                 int n_tokens, float* out, int accumulate,
                                 float* router_score_out, int* topk_i_out, float* topk_w_out,
                                 moe_b200_stream stream);

/* The same block with the RMSNorm in front of it fused in (src/forward.cpp:315 +
 * 317-514: rmsnorm(s->t, x, rms_ffn_w) followed by the MoE block, and with
 * accumulate != 0 and out == x the residual add behind it, src/forward.cpp:514).
 *   x            device f32 [n_tokens, H]: the residual stream, NOT normalised
 *   rms_weight   device [H], f32 (the CPU engine's weights) or bf16 (the GPU
 *                engine's, include/model.hpp:92) by rms_weight_dtype
 * The norm follows the CPU engine's arithmetic exactly (src/run.cpp:306-319:
 * float squares summed in double, eps 1e-5, 1.0f / sqrtf, weight * (scale * x) in
 * double rounded to float); the result is rounded to bf16 as the block input
 * always is (src/hip/BLAS.hip:32-40).  out may alias x (every read of x happens in
 * the first kernel of the call).  Other arguments as moe_b200_forward. */
moe_b200_status moe_b200_forward_norm(moe_b200_handle h, int layer, const float* x,
                                      const void* rms_weight, int rms_weight_dtype, int n_tokens,
                                      float* out, int accumulate, float* router_score_out,
                                      int* topk_i_out, float* topk_w_out, moe_b200_stream stream);

/* Same call with HOST buffers: t (pinned or pageable) is copied to the device,
 * the block runs, out is copied back, and the call returns when out is valid.
 * This is the path an engine without device-resident activations would use and
 * the one the end-to-end figure is measured through. */
moe_b200_status moe_b200_forward_host(moe_b200_handle h, int layer, const void* t_host,
                                      int t_dtype, int n_tokens, float* out_host,
                                      int* topk_i_host, float* topk_w_host);

/* Expert-parallel communicator (replaces the peer-access / peer-copy set-up of
 * src/getp/run.cpp:186-202,237-318).  Rank 0 calls moe_b200_ep_unique_id and
 * sends the 128 bytes to the other ranks by any host channel; every rank then
 * calls moe_b200_ep_init.  Uses NCCL (ncclCommInitRank) over NVLink. */
moe_b200_status moe_b200_ep_unique_id(char id_out[128]);
moe_b200_status moe_b200_ep_init(moe_b200_handle h, const char id[128]);

/* Peer-memory mode of the expert-parallel exchange (optional, instead of
 * moe_b200_ep_init): the ranks map each other's exchange buffers (CUDA IPC over
 * NVLink) and the exchange happens inside the plan / permute kernels, the expert
 * GEMMs and the combine kernel -- no NCCL call, no host wait, no extra launch.  Every rank calls
 * moe_b200_ep_peer_export, the ranks exchange the blobs by any host channel, and
 * every rank passes all of them, in rank order, to moe_b200_ep_peer_enable.  All
 * ranks must be processes on one node whose GPUs have peer access, created with
 * the same hidden_dim, n_experts, experts_per_token, max_tokens and ep_size: the
 * blobs carry these and a mismatch is refused with MOE_B200_ERR_INVALID before
 * anything is mapped (peers store into each other's buffers at addresses they
 * compute from their own configuration).  (The
 * reference enables peer access between all pairs at start-up too,
 * src/getp/run.cpp:186-202.) */
#define MOE_B200_EP_IPC_BYTES 64
#define MOE_B200_EP_PEER_EXPORT_BYTES (4 * MOE_B200_EP_IPC_BYTES)
moe_b200_status moe_b200_ep_peer_export(moe_b200_handle h, char* blob_out);
moe_b200_status moe_b200_ep_peer_enable(moe_b200_handle h, const char* all_blobs);

/* Call counter of the peer-memory exchange on this rank (the value its flags
 * carry), and the way to re-align the ranks after a call that some of them did
 * not make: every rank passes the same `sequence`, at least as large as every
 * rank's current counter, with no call in flight.  (The reference has no
 * recovery path: a failed peer copy exits the process, include/model.hpp:8-17.) */
int moe_b200_ep_peer_sequence(moe_b200_handle h);
moe_b200_status moe_b200_ep_peer_resync(moe_b200_handle h, int sequence);

/* The host-side plan of one expert-parallel exchange, as moe_b200_forward
 * computes it: cnt_all [ep_size, n_experts] holds every rank's per-expert row
 * counts (rows are sent sorted by global expert); the outputs, each [ep_size],
 * give how many rows this rank sends to / receives from each peer and the
 * first row of each peer's range in its send / receive buffer.  Pure host
 * arithmetic (replaces the per-shard bookkeeping of src/forward.cpp:565-592). */
void moe_b200_ep_plan(int n_experts, int ep_size, int ep_rank, const int* cnt_all, int* send_cnt,
                      int* send_off, int* recv_cnt, int* recv_off);

/* Token grouping of the serving loop (pure host code, no GPU needed): which
 * (sequence, position) rows go into the next forward() call.  Replaces the
 * static batches of inference() (src/getp/run.cpp:661-736) and the per-step
 * compaction of generate() (src/getp/run.cpp:573-617).  The reference steps a
 * batch until EVERY sequence of it has finished, so the rows per call -- the T
 * of the MoE block -- decay; with `continuous` != 0 a slot whose sequence
 * finished is refilled at once from the shared queue and T stays at n_slots
 * until the queue drains.  continuous == 0 reproduces the reference row for row.
 *
 * One queue is shared by all ranks (threads) of a process, one batcher per rank.
 * prompt_tokens[r] / prompt_lens[r] are request r's encoded prompt (>= 1
 * token); output_tokens[r] (optional) receives its generated tokens and a
 * closing -1, max_seq_len + 1 ints (the layout of Requests.tok_gens,
 * src/getp/eval.cpp:10-40).  The arrays stay owned by the caller.
 *
 * A step: begin_step fills tokens / positions / slots (the batch_tokens,
 * batch_positions, batch_indices arguments of forward(), src/forward.cpp:202-204;
 * a slot is the sequence's KV-cache row and starts again at position 0 when it
 * is refilled) and optionally needs_sample (1 where the row has reached the end
 * of its prompt), each n_slots ints, and returns the number of rows, 0 when all
 * requests are done, -1 on misuse.  After forward() and sampling, end_step takes
 * the sampled token per row (ignored where the prompt still supplies the next
 * token) and applies the reference's rules (src/getp/run.cpp:547-571: tokens
 * 199999 / 200002 or position + 1 >= max_seq_len end a sequence). */
typedef struct moe_b200_request_queue_s* moe_b200_request_queue;
typedef struct moe_b200_batcher_s* moe_b200_batcher;
moe_b200_status moe_b200_request_queue_create(int n_requests, const int* const* prompt_tokens,
                                              const int* prompt_lens, int* const* output_tokens,
                                              int max_seq_len, moe_b200_request_queue* out);
void moe_b200_request_queue_destroy(moe_b200_request_queue q);
moe_b200_status moe_b200_batcher_create(moe_b200_request_queue q, int n_slots, int continuous,
                                        moe_b200_batcher* out);
void moe_b200_batcher_destroy(moe_b200_batcher b);
int moe_b200_batcher_begin_step(moe_b200_batcher b, int* tokens, int* positions, int* slots,
                                int* needs_sample);
moe_b200_status moe_b200_batcher_end_step(moe_b200_batcher b, const int* sampled);
/* Forward calls made, rows they carried in total, tokens generated (any pointer may be NULL). */
void moe_b200_batcher_stats(moe_b200_batcher b, long long* steps, long long* rows,
                            long long* tokens_out);

/* Bytes of device memory the handle holds (weights + workspace). */
size_t moe_b200_device_bytes(moe_b200_handle h);
/* Text of the last error on this handle (or of the last failed create when h
 * is NULL).  Never NULL. */
const char* moe_b200_last_error(moe_b200_handle h);
/* Reads AND CLEARS the device status word (synchronises the device): 0 = no
 * kernel has reported a problem since the last read; otherwise the code of the
 * first problem (0x101..0x106: a pipeline barrier of an expert GEMM timed out;
 * 0x202: an expert index out of range; 0x301: a peer's flag in the peer-memory
 * exchange, i.e. a rank that did not join the call within 2 s; 0x302: the
 * ranks' row counts would overflow a receive buffer) and MOE_B200_ERR_DEVICE.
 * The CUDA context stays usable.  After 0x301 / 0x302 the output of that call is
 * undefined and the ranks' call counters may differ: before the next
 * expert-parallel call every rank reads its status, the ranks agree on the
 * largest moe_b200_ep_peer_sequence() over any host channel, and each passes it
 * to moe_b200_ep_peer_resync(). */
moe_b200_status moe_b200_device_status(moe_b200_handle h, int* status_word);
/* Number of kernels the last moe_b200_forward launched on this handle. */
int moe_b200_last_launch_count(moe_b200_handle h);
/* Per-expert row counts of the last forward on this rank (device->host copy,
 * synchronises): counts[n_local].  For load histograms in reports. */
moe_b200_status moe_b200_last_expert_counts(moe_b200_handle h, int* counts);

/* Per-stage device timing (the reference's -f profiling flag calls functions
 * that do not exist in its tree, src/run.cpp:1208; this is the working
 * equivalent).  moe_b200_profile(h, n_calls) arms CUDA-event pairs around the
 * stages of the next n_calls forwards on the stream they run on (n_calls == 0
 * disarms); after the stream has been synchronised,
 * moe_b200_profile_read(h, call, ms) returns the milliseconds of each stage of
 * the call-th armed forward in ms[MOE_B200_N_STAGES] (0 for a stage that did
 * not run). */
#define MOE_B200_STAGE_ROUTE 0    /* router GEMM + top-k + softmax           */
#define MOE_B200_STAGE_PLAN 1     /* offsets, tile table                     */
#define MOE_B200_STAGE_PERMUTE 2  /* row gather into expert order            */
#define MOE_B200_STAGE_DISPATCH 3 /* counts all-gather + row all-to-all (EP) */
#define MOE_B200_STAGE_REGROUP 4  /* received rows grouped by expert (EP)    */
#define MOE_B200_STAGE_GEMM1 5    /* gate/up GEMM + SwiGLU                   */
#define MOE_B200_STAGE_GEMM2 6    /* down GEMM                               */
#define MOE_B200_STAGE_RETURN 7   /* result all-to-all (EP)                  */
#define MOE_B200_STAGE_COMBINE 8  /* routing-weighted combine                */
#define MOE_B200_STAGE_H2D 9      /* moe_b200_forward_host: activations in   */
#define MOE_B200_STAGE_D2H 10     /* moe_b200_forward_host: result out       */
#define MOE_B200_N_STAGES 11
moe_b200_status moe_b200_profile(moe_b200_handle h, int n_calls);
moe_b200_status moe_b200_profile_read(moe_b200_handle h, int call, float* ms);

/* MXFP4 -> bf16 on the device, checkpoint layout in, row-major bf16 out:
 * blocks [rows, G, 16], scales [rows, G] -> out [rows, 32*G] (bf16 bits).
 * Bit-exact with dequantize_fp4 for every scale byte
 * (tools/model_export/gpt-oss-20b/export_model_bin.py:95-133).  Device
 * pointers. */
moe_b200_status moe_b200_mxfp4_unpack(const uint8_t* blocks, const uint8_t* scales, long long rows,
                                      int G, uint16_t* out_bf16, moe_b200_stream stream);

/* Decodes the RESIDENT (re-tiled) weights of one local expert with the same
 * device function the GEMM main loop uses, to row-major bf16:
 * which == 1 -> [2I, H], which == 2 -> [H, I].  For bit-exactness tests of the
 * in-kernel unpack.  Device pointer out. */
moe_b200_status moe_b200_unpack_resident(moe_b200_handle h, int layer, int local_expert, int which,
                                         uint16_t* out_bf16, moe_b200_stream stream);

/* The intermediate of the last forward (ep_size == 1 only): the bf16 SwiGLU
 * output that entered the down projection, gathered back into assignment
 * order: out_bf16 device [n_tokens * K, I], row t*K + k = expert topk_i[t][k].
 * (The engine's gate_by_expert buffer, include/model.hpp:172, in token order.)
 * Lets a test separate bf16 rounding flips of this intermediate from real
 * errors. */
moe_b200_status moe_b200_last_intermediate(moe_b200_handle h, int n_tokens, uint16_t* out_bf16,
                                           moe_b200_stream stream);

/* Routing without any allocation.  (No counterpart in the reference: its
 * router, top-k and histogram kernels write into buffers that
 * copy_transformer_to_device allocated beforehand.)
 *
 * For callers that cannot allocate device memory when they need a routing
 * decision: an engine that gave its whole memory budget to its own pools during
 * warm-up and must not meet cudaMalloc's device-wide synchronisation between
 * decode steps, or a host that only lets a plug-in touch the buffers it is
 * handed.  The call needs no handle and creates nothing: router GEMM + bias,
 * top-k, softmax and the per-expert histogram / offsets run with their scratch
 * (the per-block histograms) in a fixed array inside the library image, about
 * 0.26 MB, which every GPU that loads the library holds until the process exits.
 *
 *   t                  device [n_tokens, hidden_dim], f32 or bf16
 *   w_router_bf16      device bf16 [n_experts, hidden_dim];  b_router device f32 [n_experts]
 *   topk_i_out         device i32 [n_tokens, K]   topk_w_out  device f32 [n_tokens, K]
 *   expert_counts_out  device i32 [n_experts]     rows routed to each expert
 *   expert_offsets_out device i32 [n_experts + 1] their exclusive prefix sum
 * All five outputs are required.  Limits (MOE_B200_ERR_INVALID beyond them):
 * n_tokens <= MOE_B200_ROUTE_NOALLOC_MAX_TOKENS, n_experts <=
 * MOE_B200_ROUTE_NOALLOC_MAX_EXPERTS, hidden_dim a multiple of 64 and <=
 * MOE_B200_ROUTE_NOALLOC_MAX_HIDDEN, K <= 8.
 *
 * The first call on a device looks up the array's device address and raises the
 * kernels' shared-memory limit; make that first call before any stream capture.
 * All calls on a device share the one array: it keeps the previous call's
 * contents (every entry a call reads is written by that call first, so nothing
 * has to be cleared), and two calls that overlap on the GPU -- different
 * streams, or different host threads -- race on it. */
#define MOE_B200_ROUTE_NOALLOC_MAX_TOKENS 2048
#define MOE_B200_ROUTE_NOALLOC_MAX_EXPERTS 256
#define MOE_B200_ROUTE_NOALLOC_MAX_HIDDEN 6144
moe_b200_status moe_b200_route_noalloc(const void* t, int t_dtype, int n_tokens, int hidden_dim,
                                       const void* w_router_bf16, const float* b_router,
                                       int n_experts, int experts_per_token, int* topk_i_out,
                                       float* topk_w_out, int* expert_counts_out,
                                       int* expert_offsets_out, moe_b200_stream stream);

/* Library build info, e.g. "moe_b200 0.1 sm_100a". */
const char* moe_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H */
