/* C ABI of the Qwen3-TTS streaming codec decoder: one call turns one new frame of 16 codes of every given stream into
 * `samples_per_frame` PCM samples, with nothing recomputed. What a frame needs from the past (each causal conv's last
 * (k - 1) * dilation input rows, each overlapping transposed conv's last GEMM row, each attention layer's last 72
 * frames of K and V) lives in the stream's slot of the per-stream state, which a call reads and advances.
 *
 * Replaces the decoder that `codec::build` (crates/omni-qwen3-tts/src/codec.rs:112-448) emits into the tail of the
 * reference model's `first` and `decode` programs, and the kernels those calls launch
 * (crates/omni-qwen3-tts/kernels/codec.cu:66-513). In the reference the decoder shares a sequence's lease with the
 * talker (`Seq`); here it is a model of its own: either attached to a talker model (`omni_talker_attach_codec`, after
 * which the talker's calls open, decode and close its streams themselves), or driven by the caller, who opens a stream
 * next to the talker's sequence and hands `omni_codec_decode` the frame `omni_talker_step` returned. Weight layout transforms and scale folding happen on
 * the host at create, as `build` does at load.
 *
 * One model per GPU per thread; no internal locking; calls are synchronous. All functions return an omni_status
 * (include/omni_b200.h); after a non-zero status `omni_codec_last_error` describes it. */
#ifndef OMNI_B200_CODEC_H
#define OMNI_B200_CODEC_H

#include <stddef.h>
#include <stdint.h>

#include "omni_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* `config::Codec` (crates/omni-qwen3-tts/src/config.rs:51-67) followed by the limits of this model. Supported, as in
 * `build` (codec.rs:113-133): 16 quantizers, head_dim 64, sliding_window 72, hidden_size a multiple of 256 up to 1024,
 * latent_dim a multiple of 8 up to 8192, an output conv width (decoder_dim >> n_upsample_rates) that is a multiple of
 * 32 up to 128, a samples-per-frame count that is a multiple of 64; further, of this library's GEMMs: codebook_dim,
 * latent_dim, hidden_size, intermediate_size and heads * 64 multiples of 64, every other channel count a multiple of 8. */
typedef struct omni_codec_config {
  int32_t codebook_size, codebook_dim, latent_dim, decoder_dim, hidden_size, intermediate_size;
  int32_t num_hidden_layers, num_attention_heads, head_dim;
  float rms_norm_eps, rope_theta;
  int32_t sliding_window, num_quantizers;
  int32_t n_upsampling_ratios;
  int32_t upsampling_ratios[4]; /* the x2 stages: transposed conv (kernel = stride) + ConvNeXt */
  int32_t n_upsample_rates;
  int32_t upsample_rates[8];    /* the decoder blocks: SnakeBeta, transposed conv (kernel = 2 * rate), 3 residual units */
  int32_t max_batch;            /* streams per call */
  int32_t max_streams;          /* state slots */
  int32_t use_graphs;           /* 1: a call's kernels replayed as one CUDA graph per bucket; 0: launched one by one */
} omni_codec_config;

typedef struct omni_codec omni_codec;
typedef struct omni_codec_stream omni_codec_stream;

/* Replaces the load half of `codec::build`. Tensors by checkpoint name (f32 or bf16, host or device), the names and
 * shapes `build` reads: decoder.quantizer.{rvq_first,rvq_rest}.vq.layers.{i}._codebook.{embedding_sum,cluster_usage},
 * decoder.quantizer.{rvq_first,rvq_rest}.output_proj.weight, decoder.pre_conv.conv.{weight,bias},
 * decoder.pre_transformer.{input_proj,output_proj}.{weight,bias}, decoder.pre_transformer.layers.{i}.*,
 * decoder.pre_transformer.norm.weight, decoder.upsample.{i}.{0.conv,1.dwconv.conv,1.norm,1.pwconv1,1.pwconv2}.*,
 * decoder.upsample.{i}.1.gamma, decoder.decoder.0.conv.*, decoder.decoder.{i}.block.{0,1,2,3,4}.*,
 * decoder.decoder.{n}.{alpha,beta}, decoder.decoder.{n+1}.conv.* (codec.rs:134-407). */
int32_t omni_codec_create(const omni_codec_config* config, const omni_tensor* tensors, int32_t n_tensors, int32_t device,
                          omni_codec** out);
void omni_codec_destroy(omni_codec* m);
const char* omni_codec_last_error(const omni_codec* m);

/* A zeroed state slot: rows before the stream's start read as zero, the convs' causal padding (what a fresh lease is
 * in the reference, codec.cu:18-19). OMNI_DENIED_BUSY when every slot is taken. */
int32_t omni_codec_open(omni_codec* m, omni_codec_stream** out);
int32_t omni_codec_close(omni_codec* m, omni_codec_stream* s);
/* Frames decoded so far (the `pos` the next call runs at). */
int32_t omni_codec_stream_frames(const omni_codec_stream* s);

/* Runs every bucket (1, 2, 4, ..., max_batch) on the padding slot so that the GEMM plans exist and the graphs are
 * captured before live traffic. */
int32_t omni_codec_warmup(omni_codec* m);

/* The decoder calls of one `first` / `decode` program: codes [n][16] (the frame of each stream; a codebook-0 code past
 * the book, the talker's end of speech, reads as code 0) -> wav [n][samples_per_frame] f32 in [-1, 1] (`Out::wav`).
 * Every stream advances by one frame. Streams must be distinct. The rows between n and its bucket run on the padding
 * slot. */
int32_t omni_codec_decode(omni_codec* m, int32_t n, omni_codec_stream* const* streams, const int32_t* codes, float* wav);

/* Puts the decoder behind a talker model (include/omni_b200.h), as `codec::build` appends it to the reference model's
 * `first` and `decode` programs: from then on `omni_talker_open` / `omni_talker_close` also take and return a decoder
 * slot, and `omni_talker_start`, `omni_talker_step` and `omni_talker_step_end` decode the frames they return and fill
 * `wav` (`Out::wav`, 1,920 samples per sequence) instead of zero-filling it; the streams advance whether or not `wav` is
 * given. The decoder must give 1,920 samples per frame and take at least the talker's batch; both models must be on
 * one device. Attach (or detach, with NULL) while no sequence is open. `omni_talker_run_ticks` does not decode. */
int32_t omni_talker_attach_codec(omni_talker* talker, omni_codec* codec);

/* Samples per frame (the product of every rate). */
int32_t omni_codec_samples_per_frame(const omni_codec* m);

/* Device time of the last decode (CUDA events on the model's stream around its kernels, copies excluded) and the
 * kernels it launched. */
int32_t omni_codec_stats(const omni_codec* m, float* last_call_gpu_ms, int32_t* last_call_launches);

#ifdef __cplusplus
}
#endif
#endif
