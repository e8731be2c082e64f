/* C ABI of the Higgs-style speech model shell: a Qwen3 body over a paged KV, a fused eight-codebook embedding that is
 * also the output head (tied), eight independent code draws per step, and the delay pattern that decides which
 * codebooks a step draws and when a run ends.
 *
 * Replaces the model shell of crates/omni-higgs-audio/src/model.rs (`Model::{load, open, start, step, logits}`) one
 * level below its engine. Not part of this library: the waveform codec (`Model::decode`, the reference's `codec`
 * program). A decode step's kernels are captured into one CUDA graph per sequence count the second time that count
 * is seen and replayed from then on (no batch buckets, no padding rows); `start` is issued as per-op launches.
 *
 * One model per GPU per thread; no internal locking; calls are synchronous. All functions return an omni_status
 * (include/omni_b200.h); after a non-zero status `omni_higgs_last_error` describes it. */
#ifndef OMNI_B200_HIGGS_H
#define OMNI_B200_HIGGS_H

#include <stddef.h>
#include <stdint.h>

#include "omni_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define OMNI_HIGGS_CODEBOOKS 8 /* `CODEBOOKS` (crates/omni-higgs-audio/src/config.rs:12) */

/* The body's shape (`config::Stack`; body.vocab = text vocabulary), the codebook size (`VOCAB` = 1026, config.rs:13),
 * `Sampling` (model.rs:84-87) and `Limits` (model.rs:72-81). */
typedef struct omni_higgs_config {
  omni_stack_config body;
  int32_t code_vocab;
  float temperature;
  int32_t top_k;
  int32_t max_batch;  /* sequences per call */
  int32_t max_tokens; /* prompt rows per `start` */
  double kv_gib;      /* KV pool size */
  int32_t use_graphs; /* 1: the decode step's kernels replayed as one CUDA graph per bucket; 0: launched one by one */
  int32_t audio_adapter; /* 1: every layer carries a second, audio-only MLP of the same width beside its MLP (tensors
                            body.layers.{i}.audio_mlp.{gate,up,down}_proj.weight); on audio positions (the frame rows of
                            `start`'s first draw onwards, i.e. every decode step) both run on the same normed input and
                            their down projections are summed in f32 before the one bf16 rounding; text positions (the
                            prompt) use the plain MLP alone. No counterpart in the reference, whose Higgs body is the
                            plain Qwen3 stack (model.rs:339-405). 0: off */
} omni_higgs_config;

/* `Draw` (model.rs:99-104): a uniform per codebook, and the codes to take instead; force[b] < 0 in EVERY codebook means
 * "no force given": the step then takes the delay pattern's ramp (codebooks from `forced_from` on read BOC). */
typedef struct omni_higgs_draw {
  float uniforms[OMNI_HIGGS_CODEBOOKS];
  int32_t force[OMNI_HIGGS_CODEBOOKS];
  int32_t has_force; /* 0: `Draw::force` is None */
} omni_higgs_draw;

typedef struct omni_higgs omni_higgs;
typedef struct omni_higgs_seq omni_higgs_seq;

/* Replaces `Model::load` (model.rs:129-149). Tensors by checkpoint name, bf16 or f32:
 *   body.layers.{i}.{input_layernorm, post_attention_layernorm}.weight, body.layers.{i}.self_attn.{q,k,v,o}_proj.weight,
 *   body.layers.{i}.self_attn.{q,k}_norm.weight, body.layers.{i}.mlp.{gate,up,down}_proj.weight, body.norm.weight
 *   (fused at load as `Stack::load` does, crates/omni-qwen3/src/stack.rs:93-141),
 *   tied.embedding.text_embedding.weight [text_vocab, hidden],
 *   tied.embedding.modality_embeddings.0.embedding.weight [8 * code_vocab, hidden]   (model.rs:330-337). */
int32_t omni_higgs_create(const omni_higgs_config* config, const omni_tensor* tensors, int32_t n_tensors, int32_t device,
                          omni_higgs** out);
void omni_higgs_destroy(omni_higgs* m);
const char* omni_higgs_last_error(const omni_higgs* m);

/* Replaces `Model::open` (model.rs:152-163): pages for prompt + rows positions and a state slot.
 * OMNI_DENIED_BUSY / OMNI_DENIED_EXCEEDS_POOL as `kern_pool::Denied`. */
int32_t omni_higgs_open(omni_higgs* m, int32_t prompt, int32_t rows, omni_higgs_seq** out);
int32_t omni_higgs_close(omni_higgs* m, omni_higgs_seq* seq);
/* Delayed rows drawn so far (`Seq::rows`). */
int32_t omni_higgs_seq_rows(const omni_higgs_seq* seq);

/* Replaces `Model::start` (model.rs:166-187): prefill of every prompt (ids concatenated, prompt_lens[i] each, equal to
 * the length given to `open`), then the first draw. rows_out [n][8]: the delayed row of codes; ended_out [n]: 1 when the
 * delay pattern says the run has ended with this row (`Out::{rows, ended}`). */
int32_t omni_higgs_start(omni_higgs* m, int32_t n, omni_higgs_seq* const* seqs, const int32_t* ids,
                         const int32_t* prompt_lens, const omni_higgs_draw* draws, int32_t* rows_out,
                         int32_t* ended_out);
/* Runs the decode step of every bucket up to max_batch (1, 2, 4, ..., max_batch) on an internal padding lease, so
 * that every bucket's GEMM plans exist and its CUDA graph is captured before live traffic (what `Model::warmup` of
 * the duplex model does, crates/omni-personaplex/src/model.rs:202-240; the reference's Higgs shell compiles its
 * graphs through the same runtime call). */
int32_t omni_higgs_warmup(omni_higgs* m);
/* Replaces `Model::step` (model.rs:190-199): the next delayed row of every sequence. The sequences are padded up to
 * the bucket with rows on the padding lease (position 0, uniform 0.5, nothing forced). */
int32_t omni_higgs_step(omni_higgs* m, int32_t n, omni_higgs_seq* const* seqs, const omni_higgs_draw* draws,
                        int32_t* rows_out, int32_t* ended_out);

/* `Model::logits` (model.rs:258-260): bf16 [8 * code_vocab] of sequence s of the last call. */
int32_t omni_higgs_read_logits(omni_higgs* m, int32_t s, void* dst, size_t bytes);

/* Device time of the last start/step (CUDA events on the model's stream) and kernels it launched. */
int32_t omni_higgs_stats(const omni_higgs* m, float* last_call_gpu_ms, int32_t* last_call_launches);

#ifdef __cplusplus
}
#endif
#endif
