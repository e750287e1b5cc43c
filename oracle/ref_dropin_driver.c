/*
** TEST INFRASTRUCTURE, not product code.
**
** Drives the reference's UNMODIFIED optimizer (lang/lm_adam.c, with num/mat.c,
** num/vec.c and lang/gradutil.c) linked against libanni_b200.so INSTEAD of the
** reference's own backend object: the link-time substitution a maintainer
** would make.  With a GPU present gpu_available() answers 1 and
** lm_adam_step_scaled takes its device path (adam_step_gpu, lm_adam.c:452):
** gpu_malloc'd flats, aliasing, gpu_grad_sumsq, host clip/skip,
** gpu_adam_step_dev_bf16, pinned scatter of the host-resident vectors -- all
** through this library's symbols.  Built by oracle/Makefile into
** oracle/_ref/libannref_dropin.so, and a second time (-DDROPIN_FUSED) with
** lm_adam_fused_step.patch applied to a copy of lang/lm_adam.c into
** oracle/_ref/libannref_fused.so: the same trainer-side code with the one-launch
** engine behind lm_adam_step_scaled (used_gpu then returns 1 + the steps it took).
*/
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "gpu.h"
#include "mat.h"
#include "vec.h"
#include "lm_adam.h"

/*
** kinds[i]: 0 = weight matrix rows[i] x cols[i] (gradient produced on the
** device), 1 = bias / LayerNorm vector of rows[i] elements (host resident).
** p: all parameters back to back (in / out).  g: steps * n gradients.  m, v:
** moments out.  norms: last_grad_norm after each step.  Returns 0, or a
** negative code naming the stage that failed.
*/
int dropin_run(int n_t, const int *kinds, const int *rows, const int *cols, float *p,
	const float *g, float *m, float *v, int steps, double lr, double beta1, double beta2,
	double eps, double wd, double clip, double grad_scale, int bf16_prec, double *norms,
	int *used_gpu)
{
	lm_adam *opt;
	mat **w = calloc((size_t)n_t, sizeof(*w));
	mat **dw = calloc((size_t)n_t, sizeof(*dw));
	vec **wv = calloc((size_t)n_t, sizeof(*wv));
	vec **dwv = calloc((size_t)n_t, sizeof(*dwv));
	int n = 0;
	int i;
	int k;
	int s;
	int off;
	int rc = 0;

	*used_gpu = gpu_available();
	if (bf16_prec)
		gpu_set_compute_prec(GPU_PREC_BF16);
	for (i = 0; i < n_t; i++)
		n += kinds[i] ? rows[i] : rows[i] * cols[i];
	opt = calloc(1, sizeof(*opt));
	opt->slots = calloc((size_t)n, sizeof(lm_adam_slot));
	opt->segs = calloc((size_t)n_t, sizeof(lm_adam_seg));
	opt->n = n;
	opt->beta1 = beta1;
	opt->beta2 = beta2;
	opt->eps = eps;
	opt->weight_decay = wd;
	opt->grad_clip = clip;
	off = 0;
	for (i = 0; i < n_t; i++) {
		lm_adam_seg *sg = &opt->segs[opt->n_segs++];
		int cnt = kinds[i] ? rows[i] : rows[i] * cols[i];
		float *wp;
		float *gp;

		if (kinds[i]) {
			wv[i] = vec_create(cnt);
			dwv[i] = vec_create(cnt);
			wp = wv[i]->data;
			gp = dwv[i]->data;
			sg->wv = wv[i];
			sg->dwv = dwv[i];
		} else {
			w[i] = mat_create(rows[i], cols[i]);
			dw[i] = mat_create(rows[i], cols[i]);
			wp = w[i]->data;
			gp = dw[i]->data;
			sg->w = w[i];
			sg->dw = dw[i];
		}
		memcpy(wp, p + off, (size_t)cnt * sizeof(float));
		sg->off = off;
		sg->n = cnt;
		for (k = 0; k < cnt; k++) {
			opt->slots[off + k].param = &wp[k];
			opt->slots[off + k].grad = &gp[k];
		}
		off += cnt;
	}
	for (s = 0; s < steps && rc == 0; s++) {
		const float *gs = g + (size_t)s * (size_t)n;

		off = 0;
		for (i = 0; i < n_t; i++) {
			int cnt = opt->segs[i].n;

			if (kinds[i])
				memcpy(dwv[i]->data, gs + off, (size_t)cnt * sizeof(float));
			else if (dw[i]->d_data && dw[i]->on_device == MAT_DEV_ALIASED) {
				/* as the backward GEMMs do: write dW straight into the aliased flat */
				if (gpu_memcpy_h2d(dw[i]->d_data, gs + off, (size_t)cnt * sizeof(float)) != 0)
					rc = -10;
			} else
				memcpy(dw[i]->data, gs + off, (size_t)cnt * sizeof(float));
			off += cnt;
		}
		lm_adam_step_scaled(opt, lr, grad_scale);
		norms[s] = opt->last_grad_norm;
		if (opt->t != s + 1)
			rc = -11;
		if (*used_gpu && !opt->d_param && s == 0)
			rc = -12;	/* the device path was not taken */
	}
	lm_adam_sync_host(opt);
	off = 0;
	for (i = 0; i < n_t; i++) {
		int cnt = opt->segs[i].n;

		memcpy(p + off, kinds[i] ? wv[i]->data : w[i]->data, (size_t)cnt * sizeof(float));
		off += cnt;
	}
	for (i = 0; i < n; i++) {
		m[i] = opt->slots[i].m;
		v[i] = opt->slots[i].v;
	}
	{
		const char *e = gpu_debug_last_error();

		if (e && e[0]) {
			fprintf(stderr, "[dropin] pending CUDA error: %s\n", e);
			rc = rc ? rc : -13;
		}
	}
#ifdef DROPIN_FUSED
	/* built with lm_adam_fused_step.patch: every step must have gone through the one-launch engine */
	{
		extern int lm_adam_b200_steps;

		if (*used_gpu && lm_adam_b200_steps < steps && rc == 0)
			rc = -14;
		*used_gpu = *used_gpu ? 1 + lm_adam_b200_steps : 0;
		lm_adam_b200_steps = 0;
	}
#endif
	lm_adam_free(&opt);
	for (i = 0; i < n_t; i++) {
		if (w[i])
			mat_free(&w[i]);
		if (dw[i])
			mat_free(&dw[i]);
		if (wv[i])
			vec_free(&wv[i]);
		if (dwv[i])
			vec_free(&dwv[i]);
	}
	free(w);
	free(dw);
	free(wv);
	free(dwv);
	return rc;
}
