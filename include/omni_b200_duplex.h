/* C ABI of the duplex (PersonaPlex) model shell: the Helium temporal transformer over an FP8 ring KV, the depformer's
 * eight per-codebook passes, the Gumbel-max draws and the token bookkeeping of one 80 ms tick.
 *
 * Replaces the model shell of crates/omni-personaplex/src/model.rs (`Model::{load, open, start, tick}` and the debug
 * getters) one level below the engine. The waveform codec (Mimi) is not part of this library yet: the caller's codes
 * of a frame arrive through `omni_duplex_step.caller` (what `force_caller` overrides in the reference), and no PCM is
 * returned. A tick's kernels are captured into one CUDA graph per session count the second time that count is seen and
 * replayed from then on (no batch buckets, no padding rows and no `warmup` call).
 *
 * One model per GPU per thread; no internal locking; calls are synchronous. All functions return an omni_status
 * (include/omni_b200.h); after a non-zero status `omni_duplex_last_error` describes it. */
#ifndef OMNI_B200_DUPLEX_H
#define OMNI_B200_DUPLEX_H

#include <stddef.h>
#include <stdint.h>

#include "omni_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define OMNI_DUPLEX_STREAMS 17 /* text, the agent's 8 codebooks, the caller's 8 (config.rs:26) */
#define OMNI_DUPLEX_BOOKS 8
#define OMNI_DUPLEX_DRAWN 9  /* tokens drawn per step: text, then the agent's codebooks (config.rs:29) */
#define OMNI_DUPLEX_STATE 24 /* a session's token state: its next input row and 7 pending caller codes */

/* Shapes (crates/omni-personaplex/src/config.rs:5-37; head sizes are fixed: 128 for Helium, 64 for the depformer),
 * the reference's sampling (config.rs:55-69) and the limits of `Model::load` (model.rs:150-173). */
typedef struct omni_duplex_config {
  int32_t dim, layers, heads, hidden, context;
  int32_t dep_dim, dep_layers, dep_heads, dep_hidden;
  int32_t text_vocab, card;
  float norm_eps, rope_period;
  float text_temperature;
  int32_t text_top_k;
  float audio_temperature;
  int32_t audio_top_k;
  int32_t max_sessions; /* sessions per tick and leases in the pool */
  int32_t max_prefill;  /* prompt rows per `start` call */
  int32_t voice_rows;   /* rows of the optional "voices" tensor [voice_rows, dim] (0: none) */
  int32_t use_graphs;   /* 1: the tick's kernels replayed as one CUDA graph per bucket; 0: launched one by one */
  int32_t tp_rank, tp_size; /* tp_size = 2: this model is rank tp_rank (0 or 1) of a tensor-parallel pair, one process
                               and one GPU per rank (below); 0 or 1: the whole model on one GPU */
} omni_duplex_config;

/* `Step` (model.rs:98-107) without the PCM: tokens to take instead of drawing (-1 draws), the caller's codes to
 * hear instead of the encoder's (-1 hears `caller`), the encoder's codes of the caller's frame, the draw seed. */
typedef struct omni_duplex_step {
  int32_t force[OMNI_DUPLEX_DRAWN];
  int32_t force_caller[OMNI_DUPLEX_BOOKS];
  int32_t caller[OMNI_DUPLEX_BOOKS];
  uint64_t seed;
} omni_duplex_step;

typedef struct omni_duplex omni_duplex;
typedef struct omni_duplex_session omni_duplex_session;

enum omni_duplex_buffer {
  OMNI_DUPLEX_TEXT_LOGITS = 0,  /* bf16 [text_vocab] of session s   (`text_logits`, model.rs:446-448) */
  OMNI_DUPLEX_AUDIO_LOGITS = 1, /* bf16 [8, card] of session s      (`audio_logits`, model.rs:456-466) */
  OMNI_DUPLEX_ROWS = 2,         /* i32 [17]: the input row Helium read (`input_row`, model.rs:436-438) */
  OMNI_DUPLEX_DRAWN_BUF = 3     /* i32 [9]: the tick's draws */
};

/* Replaces `Model::load` (model.rs:175-262). Tensors by name, bf16 or f32 (rounded to nearest even), shapes checked:
 *   h.text_emb [text_vocab+1, dim], h.audio_emb [16*(card+1), dim], h.out_norm [dim], h.text_linear [text_vocab, dim],
 *   h.l{i}.norm1 [dim], h.l{i}.qkv [3*dim, dim], h.l{i}.o [dim, dim], h.l{i}.norm2 [dim],
 *   h.l{i}.gate_up [2*hidden, dim], h.l{i}.down [dim, hidden]                    (helium.rs:84-131)
 *   d.input [8*dep_dim, dim], d.text_emb [text_vocab+1, dep_dim], d.emb [7*(card+1), dep_dim], d.heads [8*card, dep_dim],
 *   d.l{i}.norm1 [dep_dim], d.l{i}.qkv [8*3*dep_dim, dep_dim], d.l{i}.out [8*dep_dim, dep_dim], d.l{i}.norm2 [dep_dim],
 *   d.l{i}.gate_in [8*2*dep_hidden, dep_dim], d.l{i}.gate_out [8*dep_dim, dep_hidden]   (depformer.rs:69-127)
 *   voices [voice_rows, dim] (optional). */
int32_t omni_duplex_create(const omni_duplex_config* config, const omni_tensor* tensors, int32_t n_tensors,
                           int32_t device, omni_duplex** out);
void omni_duplex_destroy(omni_duplex* m);
const char* omni_duplex_last_error(const omni_duplex* m);

/* Replaces `Model::open` (model.rs:287-296): a lease of `context` KV positions (a ring: position p in ring slot
 * p % context) and a token-state slot. OMNI_DENIED_BUSY when every lease is taken. */
int32_t omni_duplex_open(omni_duplex* m, omni_duplex_session** out);
/* Drop of `Session` (implicit in the reference). */
int32_t omni_duplex_close(omni_duplex* m, omni_duplex_session* session);
/* Helium position of the session's next step and frames run so far (`Session::pos`, `Session::frame`). */
int32_t omni_duplex_position(const omni_duplex_session* session, int32_t* pos, int64_t* frame);

/* `Model::is_cached` (model.rs:243-245): 1 when a prompt with exactly these rows (ids [rows, 17] and, when not NULL,
 * voice rows) sits in the on-device prefix cache. */
int32_t omni_duplex_is_cached(omni_duplex* m, int32_t rows, const int32_t* ids, const int32_t* voice);
/* `Model::warm_prefix` (model.rs:248-259): prefills the prompt into the prefix cache when it is not there yet, is at
 * most 256 rows long and one of the 8 cache slots is free; otherwise does nothing. */
int32_t omni_duplex_warm_prefix(omni_duplex* m, int32_t rows, const int32_t* ids, const int32_t* voice);

/* Replaces `Model::start` (model.rs:325-370): every eligible prompt is first brought into the prefix cache
 * (`warm_prefix`), sessions whose prompt is cached get its KV copied into their ring (`lm_copy_kv`), the others are
 * prefilled; then every session's first token state is written. row_counts[i] rows of session i, concatenated in
 * `ids` ([rows, 17], -1 = no token) and `voice` (per row: index into "voices" taken instead of the ids when >= 0;
 * NULL: none); init[i] = the first input row and the 7 pending caller codes (`Prompt::first`, `Prompt::pending`);
 * first_force[i] (NULL: none) = tokens the first tick takes unless its step forces them (`Prompt::first_force`,
 * model.rs:392-396). */
int32_t omni_duplex_start(omni_duplex* m, int32_t n, omni_duplex_session* const* sessions, const int32_t* row_counts,
                          const int32_t* ids, const int32_t* voice, const int32_t* init, const int32_t* first_force);

/* Tensor-parallel pair for Helium (no counterpart in the reference, which has no multi-GPU path). Rank r holds heads
 * [r * heads/2, (r+1) * heads/2) and MLP channels [r * hidden/2, (r+1) * hidden/2): its `create` is given
 *   h.l{i}.qkv     [3 * dim/2, dim]  = the q rows, the k rows and the v rows of its heads, in that order,
 *   h.l{i}.o       [dim, dim/2]      = the columns of its heads,
 *   h.l{i}.gate_up [2 * hidden/2, dim] = its gate rows, then its up rows,
 *   h.l{i}.down    [dim, hidden/2]   = its columns,
 * every other tensor whole (embeddings, norms, heads and the depformer are replicated; each rank's ring KV holds its
 * own heads only). After the o and the down projection the two ranks' partial rows are summed inside the add + norm
 * kernel that follows: plain loads from the peer's exchange buffer over NVLink, a flag word per rank, bounded waits
 * (a wait that runs out gives status OMNI_ERR_DEVICE on both ranks), no collective library on the data path.
 * Both ranks make the same calls with the same arguments; their logits and draws are bit-identical.
 * `tp_export` writes the handle (64 bytes) under which the other process maps this rank's exchange region;
 * `tp_connect` takes the other rank's. start / tick / warmup are refused until the pair is connected. */
#define OMNI_TP_HANDLE_BYTES 64
int32_t omni_duplex_tp_export(omni_duplex* m, void* handle, size_t bytes);
int32_t omni_duplex_tp_connect(omni_duplex* m, const void* peer_handle, size_t bytes);

/* Replaces `Model::warmup` (model.rs:202-240): runs the tick of every bucket up to max_sessions (1, 2, 4, ...,
 * max_sessions) on the padding lease, so that every bucket's GEMM plans exist and its CUDA graph is captured before
 * live traffic. Without it the first two ticks of a bucket pay for that (up to tens of ms). */
int32_t omni_duplex_warmup(omni_duplex* m);

/* Replaces `Model::tick` (model.rs:373-433): one step of every session given; emitted[i] = the text token spoken
 * now and the agent's frame (`Out::emitted`). The sessions are padded up to the bucket (`bucket`,
 * crates/omni-kern/src/lib.rs:97-101) with rows on an internal padding lease (position 0, nothing forced, seed 0:
 * model.rs:403-415). */
int32_t omni_duplex_tick(omni_duplex* m, int32_t n, omni_duplex_session* const* sessions,
                         const omni_duplex_step* steps, int32_t* emitted);

/* Debug getters of the last tick (model.rs:436-466); `s` is the session's index in that call. */
int32_t omni_duplex_read(omni_duplex* m, int32_t buffer, int32_t s, void* dst, size_t bytes);

/* Device time of the last start/tick (CUDA events on the model's stream) and kernels it launched. */
int32_t omni_duplex_stats(const omni_duplex* m, float* last_call_gpu_ms, int32_t* last_call_launches);

#ifdef __cplusplus
}
#endif
#endif
