/*
 * flux_cuda_qwen3_seam.c - the reference's text-encoder model functions, served by the B200 engine.
 *
 * Defines every symbol flux_qwen3.c exports (qwen3_model_load, qwen3_model_load_mmap, qwen3_model_free,
 * qwen3_forward, qwen3_encoder_load, qwen3_encoder_free, qwen3_encode_text; flux_qwen3.h:96-148) on top of
 * flux_cuda_qwen3_* from flux_cuda.h, so that building the reference with this file IN PLACE OF flux_qwen3.c
 * moves prompt encoding to the GPU. The tokenizer (flux_qwen3_tokenizer.c) is the reference's own and is
 * used unchanged. Compiled inside the reference's source tree together with flux_cuda_seam.c, whose
 * context it shares.
 *
 * Behaviour kept: model directory layout (model-0000{1,2}-of-00002.safetensors), malloc ownership of the
 * returned [seq, 7680] buffer, NULL on failure with the reason on stderr, padding of a prompt to 512 tokens
 * with its attention mask, the text progress callback (one event per layer the output depends on, then the
 * completion event, as the reference's own device-resident path reports it). The "mmap" loader is the same
 * resident load: 27 layers of 16-bit weights (5.5 GB) plus the embedding table stay in HBM.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "flux_cuda.h"
#include "flux_kernels.h"
#include "flux_qwen3.h"

flux_cuda_ctx *flux_cuda_seam_context(void); /* flux_cuda_seam.c */

struct qwen3_model {
  flux_cuda_qwen3 *enc;
  int num_layers;
};

qwen3_model_t *qwen3_model_load(const char *model_dir) {
  flux_cuda_ctx *ctx = flux_cuda_seam_context();
  if (!ctx || !model_dir) return NULL;
  qwen3_model_t *m = (qwen3_model_t *)calloc(1, sizeof(*m));
  if (!m) return NULL;
  if (flux_cuda_qwen3_load_dir(ctx, model_dir, QWEN3_MAX_SEQ_LEN, &m->enc) != FLUX_CUDA_OK) {
    fprintf(stderr, "qwen3_model_load: %s\n", flux_cuda_last_error());
    free(m);
    return NULL;
  }
  m->num_layers = QWEN3_NUM_LAYERS;
  return m;
}

qwen3_model_t *qwen3_model_load_mmap(const char *model_dir) { return qwen3_model_load(model_dir); }

void qwen3_model_free(qwen3_model_t *model) {
  if (!model) return;
  flux_cuda_qwen3_free(model->enc);
  free(model);
}

float *qwen3_forward(qwen3_model_t *model, const int *input_ids, const int *attention_mask, int seq_len) {
  if (!model || !model->enc || !input_ids || seq_len < 1) return NULL;
  float *out = (float *)malloc((size_t)seq_len * QWEN3_TEXT_DIM * sizeof(float));
  if (!out) return NULL;
  if (flux_cuda_qwen3_forward(model->enc, input_ids, attention_mask, seq_len, out) != FLUX_CUDA_OK) {
    fprintf(stderr, "qwen3_forward: %s\n", flux_cuda_last_error());
    free(out);
    return NULL;
  }
  if (flux_text_progress_callback) {
    for (int l = 0; l <= QWEN3_OUTPUT_LAYER_3; ++l) flux_text_progress_callback(l, model->num_layers);
    flux_text_progress_callback(model->num_layers - 1, model->num_layers);
  }
  return out;
}

qwen3_encoder_t *qwen3_encoder_load(const char *model_dir, int use_mmap) {
  if (!model_dir) return NULL;
  qwen3_encoder_t *enc = (qwen3_encoder_t *)calloc(1, sizeof(*enc));
  if (!enc) return NULL;
  char path[1024];
  snprintf(path, sizeof(path), "%s/tokenizer/tokenizer.json", model_dir);
  enc->tokenizer = qwen3_tokenizer_load(path);
  if (!enc->tokenizer) {
    fprintf(stderr, "qwen3_encoder_load: failed to load tokenizer\n");
    free(enc);
    return NULL;
  }
  snprintf(path, sizeof(path), "%s/text_encoder", model_dir);
  enc->model = use_mmap ? qwen3_model_load_mmap(path) : qwen3_model_load(path);
  if (!enc->model) {
    fprintf(stderr, "qwen3_encoder_load: failed to load model\n");
    qwen3_tokenizer_free(enc->tokenizer);
    free(enc);
    return NULL;
  }
  return enc;
}

void qwen3_encoder_free(qwen3_encoder_t *enc) {
  if (!enc) return;
  qwen3_tokenizer_free(enc->tokenizer);
  qwen3_model_free(enc->model);
  free(enc);
}

float *qwen3_encode_text(qwen3_encoder_t *enc, const char *prompt) {
  if (!enc || !enc->tokenizer || !enc->model || !prompt) return NULL;
  int n = 0;
  int *tokens = qwen3_tokenize_chat(enc->tokenizer, prompt, &n, QWEN3_MAX_SEQ_LEN);
  if (!tokens) return NULL;
  int *mask = (int *)malloc(QWEN3_MAX_SEQ_LEN * sizeof(int));
  int *padded = mask ? qwen3_pad_tokens(tokens, n, QWEN3_MAX_SEQ_LEN, mask) : NULL;
  free(tokens);
  float *emb = padded ? qwen3_forward(enc->model, padded, mask, QWEN3_MAX_SEQ_LEN) : NULL;
  free(padded);
  free(mask);
  return emb;
}
