/*
** Host-side optimizer object with the reference's interface (lang/lm_adam.h of
** the reference project) over the packed-arena engine of anni_b200.h.
**
** Same life cycle, field names and step semantics as the reference's lm_adam:
** create from the model's tensors in a fixed order, zero_grad, step /
** step_scaled (lr <= 0 is a no-op; t is incremented first, also when the step
** is then skipped; a non-finite gradient norm skips the update, zeroes the
** gradients and logs one line; last_grad_norm holds the pre-clip norm),
** invalidate, sync_host, set_offload, free.  Callers poke the hyper-parameter
** fields directly, as they do with the reference's struct.
**
** Differences, all on purpose:
**  - the tensor list is passed in as an array (the reference walks its `lm`
**    model struct, lang/lm_adam.c:117-136; the caller lists w_head, b_head, the
**    embedding when untied, then each block's tensors in that order), each tensor
**    with a decay / twin flag;
**  - parameters, gradients and moments live in device flats for good (bias and
**    LayerNorm vectors included: the reference re-uploads those every step,
**    lang/lm_adam.c:361-429); host copies are refreshed by sync_host;
**  - gradients may be bf16 and moments bf16;
**  - there is no host fallback: when the device step cannot run, the call
**    returns an error code and leaves the state untouched.
*/
#ifndef ANNI_LM_ADAM_H__
#define ANNI_LM_ADAM_H__

#include <stddef.h>
#include <stdint.h>
#include "anni_b200.h"
#include "anni_gpu_compat.h"

#ifdef __cplusplus
extern "C" {
#endif

/* One tensor of the model: host weights, host gradients (may be NULL), element count, ANNI_SEG_* flags. */
typedef struct anni_lm_tensor {
	float		*w;	/* host weights, n floats (read at first step / after invalidate, written by sync_host) */
	float		*dw;	/* host gradients, n floats, or NULL when gradients are produced on the device */
	int64_t		n;
	uint32_t	flags;
} anni_lm_tensor;

/* Mirrors lm_adam_seg (lang/lm_adam.h:21-29): where a tensor sits in the flats. */
typedef struct anni_lm_adam_seg {
	float		*w;
	float		*dw;
	int64_t		off;
	int64_t		n;
	uint32_t	flags;
	anni_mat	*w_mat;	/* trainer matrices whose device twins are views into the flats, or NULL */
	anni_mat	*dw_mat;
} anni_lm_adam_seg;

/* Mirrors lm_adam (lang/lm_adam.h:31-54); same names where the field exists there. */
typedef struct anni_lm_adam {
	anni_lm_adam_seg	*segs;
	int		n_segs;
	int64_t		n;
	int		t;
	double		beta1;
	double		beta2;
	double		eps;
	float		*h_m;		/* host mirrors of m / v as fp32 (checkpoint staging) */
	float		*h_v;
	float		*d_param;	/* device flats */
	void		*d_param_bf16;
	void		*d_param_fp8;
	void		*d_grad;
	void		*d_m;
	void		*d_v;
	int		dev_mv;		/* 1: d_m/d_v newer than h_m/h_v */
	int		params_valid;	/* 1: d_param mirrors the weights */
	int		offload_mv;	/* keep m/v on the host between steps */
	double		weight_decay;
	double		grad_clip;
	double		last_grad_norm;
	/* beyond the reference */
	int		grad_dtype;	/* ANNI_DT_* */
	int		state_dtype;
	int		last_skipped;
	int		last_error;	/* ANNI_E_* of the last step, 0 if it ran */
	double		loss_scale;	/* > 0: gradients arrive multiplied by this; folded into grad_scale */
	int		exact_update;	/* 1: ANNI_STEP_EXACT_UPDATE (default with fp32 moments) */
	void		*snap_m;	/* pinned staging and side stream of an in-flight snapshot */
	void		*snap_v;
	void		*snap_stream;
	void		*snap_event;
	size_t		grad_arena_bytes;	/* > 0: d_grad is compressible memory of this mapped size (anni_arena_alloc) */
	anni_optstep	*engine;
} anni_lm_adam;

/* lm_adam_create (lang/lm_adam.c:79): defaults beta1 0.9, beta2 0.999, eps 1e-8, wd 0, clip 0, t 0. */
anni_lm_adam	*anni_lm_adam_create(const anni_lm_tensor *tensors, int n_tensors, int grad_dtype,
			int state_dtype);
/* lm_param_count (lang/lm_adam.c:59) from the model dimensions. */
int64_t	anni_lm_param_count(int d_model, int d_ff, int n_blocks, int vocab, int tied);
void	anni_lm_adam_free(anni_lm_adam **opt);
/* lm_adam_zero_grad (lang/lm_adam.c:196): zero host gradients and the device flat. */
void	anni_lm_adam_zero_grad(anni_lm_adam *opt);
/* lm_adam_step / lm_adam_step_scaled (lang/lm_adam.c:517, :522). Return ANNI_OK or ANNI_E_*. */
int	anni_lm_adam_step(anni_lm_adam *opt, double lr);
int	anni_lm_adam_step_scaled(anni_lm_adam *opt, double lr, double grad_scale);
/* lm_adam_invalidate (lang/lm_adam.c:203): the next step re-reads the host weights. */
void	anni_lm_adam_invalidate(anni_lm_adam *opt);
/* lm_adam_sync_host (lang/lm_adam.c:336): weights into the tensors' host arrays, m/v into h_m/h_v. */
int	anni_lm_adam_sync_host(anni_lm_adam *opt);
/* lm_adam_set_offload (lang/lm_adam.c:211): pull m/v to the host and free their device flats after each step. */
void	anni_lm_adam_set_offload(int on);
/* Upload the host gradient arrays (tensors with dw != NULL) into the device flat: seg_gather's job. */
int	anni_lm_adam_upload_grads(anni_lm_adam *opt);
/*
** Hand-off with the forward / backward pass, as the reference does it (lang/lm_adam.c:239-282):
** the device twin of a weight matrix and of its gradient become VIEWS into the optimizer's
** flats (d_data = d_param + off resp. d_grad + off, on_device = aliased), so the backward GEMMs
** accumulate dW straight into the gradient flat and the step updates the weights in place -- no
** gather, no scatter.  prepare allocates the flats and uploads the weights ahead of the first
** step (gpu_buffers_init); alias attaches one tensor (gradients must be fp32 to alias dw; pass
** dw = NULL otherwise); free pulls the weights back to the host arrays and detaches every view
** (unalias_segs, lang/lm_adam.c:146-165), so the trainer never frees a slice of a flat.
*/
int	anni_lm_adam_prepare(anni_lm_adam *opt);
int	anni_lm_adam_alias(anni_lm_adam *opt, int tensor, anni_mat *w, anni_mat *dw);
/*
** The same for a bias or LayerNorm VECTOR, which the reference keeps on the host and moves twice
** per step (seg_gather / seg_scatter, lang/lm_adam.c:361-429: the "~1.8 ms of small copies" its
** own audit names): after this call the tensor's gradient lives in the device flat only.  What the
** host vector holds at that moment is uploaded once, the step stops uploading it, and (fp32
** gradients) the host vector's address is remembered so that gpu_mat_col_sum_add -- the call the
** backward pass makes with that address, num/gpu.h:198 -- adds its column sums straight into the
** flat (the reference's per-vector device accumulators, colsum_flush_all, num/gpu_cuda.cu:3142,
** without the flush).  d_w / d_dw (may be NULL) receive the device addresses of the tensor's
** weights and gradients for producers that write them directly.  Call after anni_lm_adam_prepare.
*/
int	anni_lm_adam_alias_vec(anni_lm_adam *opt, int tensor, float **d_w, void **d_dw);
/*
** Snapshot of m and v for a checkpoint without stalling the step stream (the reference's offload
** copies synchronously, lang/lm_adam.c:314-334): begin queues device-to-host copies into pinned
** staging on a side stream that first waits for the work queued so far; finish waits for them
** and converts into h_m / h_v (fp32, arena order).  Steps may be queued between the two calls
** only if they do not touch m / v before finish -- i.e. overlap it with the next forward/backward.
*/
int	anni_lm_adam_snapshot_begin(anni_lm_adam *opt);
int	anni_lm_adam_snapshot_finish(anni_lm_adam *opt);
/* Load m/v (fp32, arena order) e.g. from a checkpoint; uploaded at the next step. */
int	anni_lm_adam_set_moments(anni_lm_adam *opt, const float *m, const float *v);

/*
** Gradient-buffer helpers of lang/gradutil.h on the reference's mat / vec layout: mat_zero
** (gradutil.c:8), mat_zero_dev (:29: host and device twin together, an aliased view stays
** aliased), vec_zero (:52), mat_axpy (:58; here the device part only -- there is no host loop).
** The backward-pass GEMM wrappers of that header (mat_outer_add, mat_mul_at, mat_mul_wt*) are not
** part of the optimizer step and are not provided.
*/
void	anni_mat_zero(anni_mat *m);
void	anni_mat_zero_dev(anni_mat *m);
void	anni_vec_zero(anni_vec *v);
int	anni_mat_axpy(anni_mat *y, double a, const anni_mat *x);

/* lm_train_step_lr (lang/lm_train.c:98-124): warm-up, then "none" | "linear" | cosine decay. */
double	anni_lr_schedule(double base_lr, int step, int warmup_steps, int decay_steps,
		const char *decay_kind, int sched_from);

/*
** Adam section of a checkpoint (lang/lm_serialize.c:316-319, :263-296): int32
** {1, epoch, step, t, n}, then n interleaved (m, v) fp32 pairs in arena order,
** written through a 16 MB staging buffer.  `append` adds it after an existing
** weight section; otherwise the file is created through PATH.tmp + rename
** (lang/lm_serialize.c:298-331).  read: `offset` is the byte offset of the
** header, or -1 to take the trailer (the last 20 + 8 n bytes of the file).
*/
int	anni_ckpt_write_adam(const char *path, int append, int epoch, int step, int t, int64_t n,
		const float *m, const float *v);
int	anni_ckpt_read_adam(const char *path, int64_t offset, int64_t n_expected, int *epoch,
		int *step, int *t, float *m, float *v);

/*
** Whole checkpoints of the reference trainer (weight section + Adam section,
** lang/lm_serialize.c:103-126, :302-331, :526-587), in and out of the optimizer's flat order
** (w_head, b_head, [embedding], blocks: lang/lm_adam.c:117-136).  kind: 0 = LMCF byte-level
** model, 1 = LMCV (BPE merge table embedded), 2 = LMCT (BPE + tied embedding).  `merges` holds
** n_merges {left, right} int32 pairs (lang/bpe.c:383-401); merges_word is the count as stored,
** including the tokenizer's whitespace-runs flag bit.
*/
typedef struct anni_ckpt_model {
	int	kind;
	int	d_model;
	int	n_heads;
	int	d_ff;
	int	max_ctx;
	int	n_blocks;
	int	vocab;
	int	tied;
	int	n_merges;
	int	merges_word;
	int64_t	n;		/* optimizer slots implied by the dimensions (lm_param_count) */
	int	has_adam;
	int	epoch;
	int	step;
	int	t;
} anni_ckpt_model;

/* Header, slot count and Adam header of a checkpoint file; nothing else is read. */
int	anni_ckpt_probe(const char *path, anni_ckpt_model *info);
/*
** lm_load_checkpoint / lm_load: weights into w[info->n] in optimizer order, m and v (may be
** NULL) likewise, the merge pairs into merges (may be NULL).  Shapes in the file must match the
** header's dimensions, the Adam slot count must match the model.
*/
int	anni_ckpt_load(const char *path, anni_ckpt_model *info, float *w, float *m, float *v,
		int32_t *merges);
/*
** lm_save_checkpoint (m, v given: has_adam = 1 with info's epoch, step, t) or lm_save (m = v =
** NULL: has_adam = 0), byte-identical to the reference's files; written to PATH.tmp and renamed.
*/
int	anni_ckpt_save(const char *path, const anni_ckpt_model *info, const int32_t *merges,
		const float *w, const float *m, const float *v);

#ifdef __cplusplus
}
#endif

#endif
