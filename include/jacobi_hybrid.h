/* jacobi_hybrid.h — C ABI of libjf_hybrid.so: layered hybrid decoders (softmax attention with a sink whose values are
 * its keys, selective scans, gated delta rule layers, squared-ReLU feed-forward; one norm per layer feeding mixer and
 * feed-forward side by side) on B200.
 *
 * Same conventions as jacobi_b200.h: every function returns 0 or a negative status, hy_last_error(h) gives the text,
 * plain pointers and sizes only, host buffers are caller-owned, device memory belongs to the handle, one host thread per
 * handle.  There is no CPU fallback: without a CUDA device hy_create fails.
 *
 * A model is a list of layers (hy_layer_cfg) over a shared residual stream.  The host names tensors as the checkpoint
 * does ("l<i>.norm1", "l<i>.mix.left.q", ...); merging of the projections that read the same input and the layouts the
 * kernels want are made behind hy_finalize.  A step runs a batch of entries, each the next tokens of one request (a
 * portion of a prompt or a single decoded token), against the paged key cache and the request's recurrent-state slot.
 */
#ifndef JACOBI_HYBRID_H_
#define JACOBI_HYBRID_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hy_engine* hy_handle;

typedef enum { HY_OK = 0, HY_ERR_INVALID = -1, HY_ERR_CUDA = -2, HY_ERR_CAPACITY = -3, HY_ERR_UNSUPPORTED = -4 } hy_status;
typedef enum { HY_DTYPE_BF16 = 0, HY_DTYPE_F32 = 1, HY_DTYPE_F16 = 2, HY_DTYPE_I32 = 3 } hy_dtype;
typedef enum { HY_MIX_ATTN_SCAN = 0, HY_MIX_DELTA = 1 } hy_mixer_kind;
typedef enum { HY_FF_NONE = 0, HY_FF_RELU2 = 1 } hy_ff_kind;

typedef struct {
  int32_t mixer;                   /* hy_mixer_kind */
  /* HY_MIX_ATTN_SCAN, attention side: query heads, key heads (values are the keys), key size, value size, conv taps,
   * the query temperature 1 + qt_coef * ln(floor((p + 1) / qt_every) + 1), the score scale */
  int32_t a_heads, a_kv_heads, a_dim, a_vdim, a_conv, a_qt_every;
  float a_scale, a_qt_coef;
  /* scan side: channels, state size, rank of the step-size projection, conv taps */
  int32_t s_inner, s_state, s_dt_rank, s_conv;
  float left_scale, right_scale;   /* mixer = left_scale * attention + right_scale * scan */
  /* HY_MIX_DELTA: value heads, query/key heads, key size, value size, conv taps, inner sizes of the two-step decay and
   * gate projections (read from the tensor shapes) */
  int32_t d_heads, d_kv_heads, d_dim, d_vdim, d_conv, d_low_a, d_low_g;
  int32_t ff_kind, ff;             /* hy_ff_kind, hidden size of the feed-forward */
} hy_layer_cfg;

typedef struct {
  int32_t width, vocab, n_layers;
  int32_t dtype;                   /* HY_DTYPE_BF16: bf16 operands, fp32 accumulation / state / residual; HY_DTYPE_F32: all fp32 */
  float emb_scale, logit_scale, norm_eps;
} hy_model_cfg;

typedef struct {
  int32_t device;
  int32_t max_step_tokens;         /* tokens of all entries of one step */
  int32_t max_step_entries;
  int32_t page_size;               /* tokens per key-cache page (multiple of 16) */
  int32_t num_pages;
  int32_t max_pages_per_seq;
  int32_t num_slots;               /* recurrent-state slots (one per live request) */
  int32_t max_want;                /* rows whose logits one step may return */
} hy_runtime_cfg;

int hy_create(const hy_model_cfg* model, const hy_layer_cfg* layers, const hy_runtime_cfg* rt, hy_handle* out);
void hy_destroy(hy_handle h);
const char* hy_last_error(hy_handle h);

/* One checkpoint tensor by name (host pointer).  All tensors first, then hy_finalize. */
int hy_load_tensor(hy_handle h, const char* name, const void* data, const int64_t* shape, int32_t ndim, int32_t dtype);
int hy_finalize(hy_handle h);

/* One step.  tokens[total] holds the entries' tokens back to back; entry e covers [ent_start[e], ent_start[e+1]) and its
 * first token sits at position ent_pos0[e] of its request (the positions before it are in the cache / state already; an
 * entry with ent_pos0 == 0 starts from the empty state whatever its slot held).  pages[e * max_pages_per_seq + i] is the
 * page of tokens [i * page_size, (i + 1) * page_size).  want[n_want] are indices into tokens[]; logits_out (host, fp32,
 * [n_want, vocab]) and sampled_out (host, int32 [n_want]) may be NULL.  temperature[n_want] NULL or 0 = argmax, else a
 * draw from softmax(logits / temperature) with the counter-based generator keyed by (seed, want index).
 * layers_out: NULL, or host fp32 [n_layers, total, width] receiving the residual stream after every layer. */
int hy_step(hy_handle h, int32_t n_entries, const int32_t* tokens, const int32_t* ent_start, const int32_t* ent_pos0,
            const int32_t* ent_slot, const int32_t* pages, int32_t n_want, const int32_t* want, float* logits_out,
            int32_t* sampled_out, const float* temperature, uint64_t seed, float* layers_out);

int64_t hy_launch_count(hy_handle h);
/* Device milliseconds of the last hy_step (CUDA events on the handle's stream). */
float hy_last_step_ms(hy_handle h);
/* Bytes of device memory held: weights, cache pages, state slots, workspace. */
int hy_memory_info(hy_handle h, int64_t* weights, int64_t* cache, int64_t* state, int64_t* workspace);

/* Device time per group of kernels, summed over the steps since hy_profile_enable(h, 1): ms[HY_PROFILE_CATEGORIES]. */
enum { HY_PROF_NORM = 0, HY_PROF_GEMM_IN = 1, HY_PROF_CONV = 2, HY_PROF_ATTN = 3, HY_PROF_SMALL_GEMM = 4, HY_PROF_SCAN = 5,
       HY_PROF_DELTA = 6, HY_PROF_GEMM_OUT = 7, HY_PROF_HEAD = 8, HY_PROFILE_CATEGORIES = 9 };
int hy_profile_enable(hy_handle h, int32_t on);
int hy_profile_read(hy_handle h, float* ms);

#ifdef __cplusplus
}
#endif
#endif
