/*
** TEST INFRASTRUCTURE, not product code.
**
** Thin driver around the UNMODIFIED reference sources (lang/lm_adam.c,
** lang/lm_train.c, lang/lm_serialize.c linked with num/gpu_stub.c).  It is
** compiled by oracle/Makefile against the reference headers where they lie and
** the result goes to oracle/_ref/libannref.so.  Nothing here restates any
** arithmetic: every number these entry points return was computed by the
** reference's own object code.  They exist so that Python (ctypes) can
**   - pin oracle/oracle_adam.c against the reference bit for bit,
**   - generate the golden vectors under tests/golden/,
**   - time the reference's CPU step as bench.py's "reference" arm.
*/
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "lm.h"
#include "lm_adam.h"
#include "lm_train.h"
#include "lm_serialize.h"

/*
** One lm_adam_step_scaled() (lang/lm_adam.c:522) over caller arrays.  The
** public lm_adam struct (lang/lm_adam.h:31-54) is filled by hand: one slot per
** scalar pointing into p[] / g[], no segments, so the stub backend
** (gpu_available()==0) sends the call down the host loop at :559-606.
** t_before is opt->t before the call (the step increments it first).
** Returns 0, or -1 when memory ran out.
*/
int ref_adam_step(float *p, float *g, float *m, float *v, int n, int t_before,
	double lr, double beta1, double beta2, double eps, double wd, double clip,
	double grad_scale)
{
	lm_adam opt;
	int i;

	memset(&opt, 0, sizeof(opt));
	opt.slots = malloc((size_t)n * sizeof(lm_adam_slot));
	if (!opt.slots)
		return -1;
	for (i = 0; i < n; i++) {
		opt.slots[i].param = &p[i];
		opt.slots[i].grad = &g[i];
		opt.slots[i].m = m[i];
		opt.slots[i].v = v[i];
	}
	opt.n = n;
	opt.t = t_before;
	opt.beta1 = beta1;
	opt.beta2 = beta2;
	opt.eps = eps;
	opt.weight_decay = wd;
	opt.grad_clip = clip;
	lm_adam_step_scaled(&opt, lr, grad_scale);
	for (i = 0; i < n; i++) {
		m[i] = opt.slots[i].m;
		v[i] = opt.slots[i].v;
	}
	free(opt.slots);
	return opt.t == t_before + 1 ? 0 : -2;
}

/*
** Same call with the slot table kept between repeats, for timing: the table
** build (24 bytes per scalar) is set-up, the step is what a trainer pays.
*/
typedef struct ref_adam_bench {
	lm_adam	opt;
} ref_adam_bench;

void *ref_adam_bench_create(float *p, float *g, int n, double beta1,
	double beta2, double eps, double wd, double clip, int t_before)
{
	ref_adam_bench *b = calloc(1, sizeof(*b));
	int i;

	if (!b)
		return NULL;
	b->opt.slots = malloc((size_t)n * sizeof(lm_adam_slot));
	if (!b->opt.slots) {
		free(b);
		return NULL;
	}
	for (i = 0; i < n; i++) {
		b->opt.slots[i].param = &p[i];
		b->opt.slots[i].grad = &g[i];
		b->opt.slots[i].m = 0.0f;
		b->opt.slots[i].v = 0.0f;
	}
	b->opt.n = n;
	b->opt.t = t_before;
	b->opt.beta1 = beta1;
	b->opt.beta2 = beta2;
	b->opt.eps = eps;
	b->opt.weight_decay = wd;
	b->opt.grad_clip = clip;
	return b;
}

void ref_adam_bench_step(void *h, double lr, double grad_scale)
{
	ref_adam_bench *b = h;

	lm_adam_step_scaled(&b->opt, lr, grad_scale);
}

void ref_adam_bench_free(void *h)
{
	ref_adam_bench *b = h;

	if (!b)
		return;
	free(b->opt.slots);
	free(b);
}

/* lm_train_step_lr (lang/lm_train.c:98) under the given schedule settings. */
double ref_step_lr(double base_lr, int step, int warmup, int decay,
	const char *kind, int from)
{
	double lr;

	lm_train_set_lr_schedule(warmup, decay, kind);
	lm_train_set_lr_sched_from(from);
	lr = lm_train_step_lr(base_lr, step);
	lm_train_set_lr_sched_from(0);
	lm_train_set_lr_schedule(0, 0, "none");
	return lr;
}

/*
** Checkpoint written by lm_save_checkpoint (lang/lm_serialize.c:302) for a
** freshly created model of the compiled-in test dimensions: m[i], v[i] are
** placed in slots[i] (i < *n_io, which must equal the optimizer's slot count;
** pass 0 in *n_io to only query the count).  Returns 0 on success.
*/
int ref_ckpt_save(const char *path, int vocab, const float *m, const float *v,
	int *n_io, int t, int epoch, int step)
{
	lm *model;
	lm_adam *opt;
	int i;
	int rc;

	model = lm_create_vocab(vocab);
	if (!model)
		return -1;
	opt = lm_adam_create(model);
	if (!opt) {
		lm_free(&model);
		return -1;
	}
	if (*n_io == 0) {
		*n_io = opt->n;
		lm_adam_free(&opt);
		lm_free(&model);
		return 0;
	}
	if (*n_io != opt->n) {
		*n_io = opt->n;
		lm_adam_free(&opt);
		lm_free(&model);
		return -2;
	}
	for (i = 0; i < opt->n; i++) {
		opt->slots[i].m = m[i];
		opt->slots[i].v = v[i];
	}
	opt->t = t;
	rc = lm_save_checkpoint(model, opt, epoch, step, path);
	lm_adam_free(&opt);
	lm_free(&model);
	return rc;
}

/* lm_load_checkpoint (lang/lm_serialize.c:526): hand back t, epoch, step, m, v. */
int ref_ckpt_load(const char *path, float *m, float *v, int n_cap, int *n_out,
	int *t_out, int *epoch_out, int *step_out)
{
	lm *model;
	lm_adam *opt = NULL;
	int i;

	model = lm_load_checkpoint(path, &opt, epoch_out, step_out);
	if (!model || !opt)
		return -1;
	*n_out = opt->n;
	*t_out = opt->t;
	for (i = 0; i < opt->n && i < n_cap; i++) {
		m[i] = opt->slots[i].m;
		v[i] = opt->slots[i].v;
	}
	lm_adam_free(&opt);
	lm_free(&model);
	return 0;
}

/* Segment list of lm_adam_create (lang/lm_adam.c:117-136) for the compiled-in dims. */
int ref_seg_list(int vocab, int *off, int *n, int *is_vec, int cap)
{
	lm *model;
	lm_adam *opt;
	int i;
	int ns;

	model = lm_create_vocab(vocab);
	if (!model)
		return -1;
	opt = lm_adam_create(model);
	if (!opt) {
		lm_free(&model);
		return -1;
	}
	ns = opt->n_segs;
	for (i = 0; i < ns && i < cap; i++) {
		off[i] = opt->segs[i].off;
		n[i] = opt->segs[i].n;
		is_vec[i] = opt->segs[i].wv != NULL;
	}
	lm_adam_free(&opt);
	lm_free(&model);
	return ns;
}

/*
** Full checkpoints (weight section + Adam section) of the three kinds the
** reference writes (lang/lm_serialize.c:103-126): mode 0 = byte-level model
** (LMCF), 1 = BPE tokenizer embedded (LMCV), 2 = BPE + tied embedding (LMCT).
** The BPE table is synthetic: merge i joins tokens (VOCAB_SPECIALS + 2i) and
** (VOCAB_SPECIALS + 2i + 1); only its byte layout matters here.  Weights are set
** from w[] in OPTIMIZER order (the slot order of lm_adam_create) before saving.
** *n_io = 0 only queries the slot count.
*/
#include "bpe.h"

static lm *make_model(int mode, int n_merges)
{
	bpe *tok;
	int *l;
	int *r;
	int i;
	lm *model;

	if (mode == 0)
		return lm_create();
	l = malloc((size_t)(n_merges ? n_merges : 1) * sizeof(int));
	r = malloc((size_t)(n_merges ? n_merges : 1) * sizeof(int));
	for (i = 0; i < n_merges; i++) {
		l[i] = VOCAB_SPECIALS + (2 * i) % 256;
		r[i] = VOCAB_SPECIALS + (2 * i + 1) % 256;
	}
	tok = bpe_create(l, r, n_merges);
	free(l);
	free(r);
	if (!tok)
		return NULL;
	model = mode == 2 ? lm_create_bpe_tied(tok) : lm_create_bpe(tok);
	if (!model)
		bpe_free(&tok);
	return model;
}

int ref_ckpt_save_full(const char *path, int mode, int n_merges, const float *w, const float *m,
	const float *v, int *n_io, int t, int epoch, int step)
{
	lm *model = make_model(mode, n_merges);
	lm_adam *opt;
	int i;
	int rc;

	if (!model)
		return -1;
	opt = lm_adam_create(model);
	if (!opt) {
		lm_free(&model);
		return -1;
	}
	if (*n_io != opt->n) {
		rc = *n_io == 0 ? 0 : -2;
		*n_io = opt->n;
		lm_adam_free(&opt);
		lm_free(&model);
		return rc;
	}
	for (i = 0; i < opt->n; i++) {
		*opt->slots[i].param = w[i];
		opt->slots[i].m = m[i];
		opt->slots[i].v = v[i];
	}
	opt->t = t;
	rc = lm_save_checkpoint(model, opt, epoch, step, path);
	lm_adam_free(&opt);
	lm_free(&model);
	return rc;
}

/* lm_load_checkpoint, everything handed back in optimizer order. */
int ref_ckpt_load_full(const char *path, float *w, float *m, float *v, int n_cap, int *n_out,
	int *t_out, int *epoch_out, int *step_out, int *vocab_out, int *tied_out)
{
	lm *model;
	lm_adam *opt = NULL;
	int i;

	model = lm_load_checkpoint(path, &opt, epoch_out, step_out);
	if (!model || !opt)
		return -1;
	*n_out = opt->n;
	*t_out = opt->t;
	*vocab_out = model->vocab_size;
	*tied_out = model->embed->tied;
	for (i = 0; i < opt->n && i < n_cap; i++) {
		w[i] = *opt->slots[i].param;
		m[i] = opt->slots[i].m;
		v[i] = opt->slots[i].v;
	}
	lm_adam_free(&opt);
	lm_free(&model);
	return 0;
}
