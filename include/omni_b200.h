/* omni_b200.h — C ABI of the B200-native codec-frame token loop.
 *
 * One shared library, plain pointers and sizes, no C++ or framework types in
 * any signature. The entry points are what a Rust `-sys` crate (or cgo, JNI,
 * ctypes) binds in place of the reference's model shell for the Qwen3-TTS
 * talker: `Model::{load, open, start, step}` of
 * crates/omni-qwen3-tts/src/model.rs. Each declaration cites the reference
 * interface it replaces (paths relative to the reference root).
 *
 * Conventions
 *  - Every function returns an `int32_t` status: 0 is success, positive values
 *    are admission refusals a caller retries or drops (`OMNI_DENIED_*`),
 *    negative values are errors. Nothing aborts or traps; after a device-side
 *    error the model stays usable for `close` / `destroy`.
 *  - The library owns all device memory. Host arrays passed to a call are
 *    copied before the call returns; result arrays are caller-owned.
 *  - A model is bound to the thread and device that created it, like the
 *    reference's (`engine.rs:274-277`); no internal locking.
 *  - There is no CPU path: if no CUDA device is usable, `create` fails.
 */
#ifndef OMNI_B200_H
#define OMNI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OMNI_GROUPS 16 /* codebooks per frame, `GROUPS` of talker.rs:48 */
#define OMNI_PAGE 16   /* tokens per KV page, `PAGE` of omni-qwen3/src/stack.rs:30 */

enum omni_status {
  OMNI_OK = 0,
  OMNI_DENIED_BUSY = 1,         /* kern_pool::Denied::Busy: retry when sequences close */
  OMNI_DENIED_EXCEEDS_POOL = 2, /* kern_pool::Denied::ExceedsPool: can never fit */
  OMNI_ERR_INVALID = -1,        /* an argument outside its domain (model.rs:348-359) */
  OMNI_ERR_CUDA = -2,           /* a CUDA runtime/driver call failed */
  OMNI_ERR_DEVICE = -3,         /* a kernel set the device error word (bounded wait ran out, bad index) */
  OMNI_ERR_MISSING_TENSOR = -4, /* a checkpoint tensor is absent or has the wrong shape */
  OMNI_ERR_UNSUPPORTED = -5     /* a shape the kernels are not built for */
};

enum omni_dtype { OMNI_BF16 = 0, OMNI_F32 = 1 };
enum omni_location { OMNI_HOST = 0, OMNI_DEVICE = 1 };

/* One checkpoint tensor under its checkpoint name, e.g.
 * "talker.model.layers.0.self_attn.q_proj.weight". Replaces
 * `omni_kern::weights::File::expect` (crates/omni-kern/src/weights.rs:25-121);
 * f32 data is rounded to bf16 (round-to-nearest-even, lib.rs:62-66). */
typedef struct omni_tensor {
  const char* name;
  const void* data;
  int32_t dtype;    /* enum omni_dtype */
  int32_t ndim;
  int64_t shape[4];
  int32_t location; /* enum omni_location: device pointers are copied device-to-device */
} omni_tensor;

/* `omni_qwen3::config::Stack` (crates/omni-qwen3/src/config.rs:9-22). */
typedef struct omni_stack_config {
  int32_t hidden, inter, layers, q_heads, kv_heads, head_dim, vocab;
  float rms_eps, rope_theta;
} omni_stack_config;

enum omni_sampler {
  OMNI_SAMPLER_UNIFORMS = 0, /* the reference's: host-supplied uniform per draw (talker.cu:171-293) */
  OMNI_SAMPLER_PHILOX = 1    /* uniforms from Philox4x32-10 keyed by the sequence's seed, on the device */
};

/* Shapes (`config::Model`, crates/omni-qwen3-tts/src/config.rs:13-37), sampling
 * constants (`config::Generation`, :40-48) and `Limits` (model.rs:56-64). */
typedef struct omni_talker_config {
  omni_stack_config talker;    /* vocab = codec vocabulary of codebook 0 */
  omni_stack_config predictor; /* vocab = entries per residual codebook */
  int32_t groups;              /* codebooks per frame, <= OMNI_GROUPS */
  int32_t tts_pad_token_id, codec_eos_token_id;
  float temperature;
  int32_t top_k;
  float repetition_penalty;
  float sub_temperature;
  int32_t sub_top_k;
  float top_p;            /* 1.0 = off (the reference has none) */
  int32_t sampler;        /* enum omni_sampler */
  int32_t min_frames;     /* frames before the end token may be drawn (talker.rs:52) */
  int32_t control_tokens; /* top of the codec vocabulary never drawn but the end (talker.rs:54) */
  int32_t max_batch;      /* Limits::max_batch */
  int32_t max_tokens;     /* Limits::max_tokens: prompt rows per `start` */
  double kv_gib;          /* Limits::kv_gib: talker KV pool size */
  int32_t use_graphs;     /* 1: one CUDA graph per batch bucket per program; 0: eager launches */
  int32_t gemm_path;      /* 0: auto (vector GEMV for few rows, tcgen05 tiles otherwise); 1: GEMV only */
  int32_t tick_kernel;    /* 1: run each graph program as ONE persistent cooperative kernel (phase list with grid
                             barriers, weights streamed across phase boundaries) when the shapes allow it;
                             3: the same for the talker step, then ONE launch of thread-block clusters for the code
                             predictor's sub-steps (sessions dealt to clusters of 16 CTAs that never talk to one
                             another; measured slower than 1 on B200 at every session count, kept as an option);
                             0: one kernel per op */
} omni_talker_config;

/* `Draw` (model.rs:75-79): a uniform per codebook, or the frame to take
 * instead (teacher forcing); force[g] < 0 means draw. */
typedef struct omni_draw {
  float uniforms[OMNI_GROUPS];
  int32_t force[OMNI_GROUPS];
} omni_draw;

typedef struct omni_talker omni_talker;
typedef struct omni_seq omni_seq;

/* Debug buffers of the last call (model.rs:241-262). */
enum omni_buffer {
  OMNI_BUF_LOGITS = 0,   /* bf16 [vocab] of sequence s                          (`talker_logits`) */
  OMNI_BUF_P_LOGITS = 1, /* bf16 [groups-1, p_vocab] of sequence s               (`predictor_logits`) */
  OMNI_BUF_EMBEDS = 2,   /* bf16 prompt embeddings of the last `start`, leading bytes (`embeds`) */
  OMNI_BUF_HIDDEN = 3,   /* bf16 [hidden] talker hidden state of sequence s */
  OMNI_BUF_PAD_EMBED = 4 /* bf16 [hidden] */
};

typedef struct omni_stats {
  float last_call_gpu_ms; /* device time of the last start/step, CUDA events on the model's stream */
  int32_t last_call_launches; /* kernels of this library launched by the last start/step (graph nodes included) */
  int32_t bucket;             /* batch bucket the last graph call ran at */
  int32_t pages_total, pages_used;
  int64_t weight_bytes, kv_bytes;
} omni_stats;

/* Replaces `Model::load` (model.rs:111-131): takes the checkpoint's tensors,
 * fuses Q|K|V and gate|up (omni-qwen3/src/stack.rs:93-141), stacks the
 * predictor tables (talker.rs:85-93), allocates the paged KV pool and the
 * per-sequence state slots, computes the pad embedding (`Talker::init`). */
int32_t omni_talker_create(const omni_talker_config* cfg, const omni_tensor* tensors, int32_t n_tensors,
                           int32_t device, omni_talker** out);
void omni_talker_destroy(omni_talker* m);

/* Replaces `Model::open` (model.rs:135-146): leases ceil((prompt+frames)/16)
 * pages and a zeroed state slot. */
int32_t omni_talker_open(omni_talker* m, int32_t prompt_tokens, int32_t max_frames, omni_seq** out);
/* Replaces dropping a `Seq` (the lease returns to the pool). */
int32_t omni_talker_close(omni_talker* m, omni_seq* seq);
/* Seed of the sequence's Philox stream (OMNI_SAMPLER_PHILOX only). The
 * reference keeps its RNG in the engine (`Job::rng`, engine.rs:118-120). */
int32_t omni_talker_seq_seed(omni_talker* m, omni_seq* seq, uint64_t seed);
int32_t omni_talker_seq_frames(const omni_seq* seq);

/* Replaces `Model::start` (model.rs:153-177): prefill of `n` fresh sequences
 * (prompt rows concatenated in `text_ids` / `codec_ids`, codec id -1 = none)
 * and their first frame. codes: [n][16] i32. wav: [n][1920] f32 or NULL: the
 * frames' samples when a codec decoder is attached (omni_talker_attach_codec,
 * include/omni_b200_codec.h), zero-filled otherwise. */
int32_t omni_talker_start(omni_talker* m, int32_t n, omni_seq* const* seqs, const int32_t* text_ids,
                          const int32_t* codec_ids, const int32_t* prompt_lens, const omni_draw* draws,
                          int32_t* codes, float* wav);
/* Replaces `Model::step` (model.rs:180-192): one more frame per sequence. */
int32_t omni_talker_step(omni_talker* m, int32_t n, omni_seq* const* seqs, const omni_draw* draws, int32_t* codes,
                         float* wav);

/* `Model::step` in two halves, so that the engine thread can work while the GPU does (the reference's engine waits
 * on `prefill+first` and on `decode` with nothing else to do, docs/qwen3-tts.md:218-221): `step_begin` stages the
 * draws in its own pinned block, enqueues the tick and the read-back and returns; `step_end` waits for the OLDEST
 * step begun and hands out its frames. Up to two steps may be under way: a step's inputs are its draws alone (the
 * codes it needs sit in the sequences' slots on the device), so step t + 1 can be begun before step t is ended and
 * the host's staging, the copies and the engine's own work between the calls overlap the previous tick. Sequences
 * count a frame at `step_begin`. While a step is under way `start`, `step`, `run_ticks` and `close` are refused.
 * The first `step_begin` after create allocates the two pinned blocks. */
int32_t omni_talker_step_begin(omni_talker* m, int32_t n, omni_seq* const* seqs, const omni_draw* draws);
int32_t omni_talker_step_end(omni_talker* m, int32_t* codes, float* wav);

/* `ticks` back-to-back steps of the same `n` sequences with every tick's draws
 * staged in device memory before the first tick starts, so no host transfer
 * falls inside a tick. draws: [ticks][n]. codes: [ticks][n][16] or NULL.
 * tick_ms: [ticks] device time of each tick (CUDA events) or NULL. No
 * counterpart in the reference (its engine waits on every step); this is the
 * measurement entry the device-resident throughput figure uses. */
int32_t omni_talker_run_ticks(omni_talker* m, int32_t n, omni_seq* const* seqs, int32_t ticks,
                              const omni_draw* draws, int32_t* codes, float* tick_ms);

/* Replaces `Model::embeds / talker_logits / predictor_logits` (model.rs:241-262). */
int32_t omni_talker_read(omni_talker* m, int32_t buffer, int32_t s, void* dst, size_t bytes);
/* `Model::is_end` (model.rs:148-150). */
int32_t omni_talker_is_end(const omni_talker* m, const int32_t* frame);
int32_t omni_talker_stats(omni_talker* m, omni_stats* out);
/* A measurement aid with no counterpart in the reference (which is profiled with nsys from outside): names a text
 * file that receives, after every omni_talker_run_ticks call, the per-phase device timestamps of the call's last tick
 * (one line per phase of the persistent kernel: its shape, its barrier-to-barrier time, and when the first operand
 * tile, the first accumulator, the CTA's share and the barrier were reached, median and latest over the CTAs, in
 * ns). NULL or "" switches it off. The stamps cost about 1 % of a tick. */
int32_t omni_talker_trace(omni_talker* m, const char* path);
const char* omni_talker_last_error(const omni_talker* m);
/* `omni_kern::bucket` (crates/omni-kern/src/lib.rs:31-36). */
int32_t omni_bucket(int32_t n);
const char* omni_version(void);

#ifdef __cplusplus
}
#endif
#endif /* OMNI_B200_H */
