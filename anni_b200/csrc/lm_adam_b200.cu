/*
** Host-side optimizer object with the reference's interface (lang/lm_adam.c of
** the reference project) over the packed-arena engine, plus the two small host
** pieces that travel with it: the LR schedule the trainer feeds it and the Adam
** section of the checkpoint.  Plain C-style host code; every parameter update
** happens in the kernels of optstep.cu.
*/
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <atomic>
#include <chrono>
#include <thread>
#include <vector>
#include "anni_gpu_compat.h"
#include "anni_lm_adam.h"
#include "optstep_internal.h"

static int g_offload_all;

/* ---- small host helpers ------------------------------------------------------- */

static uint16_t bf16_rne_host(float x)
{
	uint32_t u;

	memcpy(&u, &x, sizeof(u));
	if ((u & 0x7fffffffu) > 0x7f800000u)
		return 0x7fffu;
	u += 0x7fffu + ((u >> 16) & 1u);
	return (uint16_t)(u >> 16);
}

static float bf16_to_f32_host(uint16_t h)
{
	uint32_t u = (uint32_t)h << 16;
	float f;

	memcpy(&f, &u, sizeof(f));
	return f;
}

static size_t elem_size(int dtype)
{
	return dtype == ANNI_DT_BF16 ? 2u : 4u;
}

/* fp32 host array -> device buffer of the given element type */
static int upload_as(void *dst, int dtype, const float *src, int64_t n)
{
	uint16_t *tmp;
	int64_t i;
	int rc;

	if (n == 0)
		return 0;
	if (dtype == ANNI_DT_F32)
		return cudaMemcpy(dst, src, (size_t)n * 4u, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -1;
	tmp = (uint16_t *)malloc((size_t)n * 2u);
	if (!tmp)
		return -1;
	for (i = 0; i < n; i++)
		tmp[i] = bf16_rne_host(src[i]);
	rc = cudaMemcpy(dst, tmp, (size_t)n * 2u, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -1;
	free(tmp);
	return rc;
}

/* device buffer of the given element type -> fp32 host array */
static int download_as(float *dst, const void *src, int dtype, int64_t n)
{
	uint16_t *tmp;
	int64_t i;

	if (n == 0)
		return 0;
	if (dtype == ANNI_DT_F32)
		return cudaMemcpy(dst, src, (size_t)n * 4u, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
	tmp = (uint16_t *)malloc((size_t)n * 2u);
	if (!tmp)
		return -1;
	if (cudaMemcpy(tmp, src, (size_t)n * 2u, cudaMemcpyDeviceToHost) != cudaSuccess) {
		free(tmp);
		return -1;
	}
	for (i = 0; i < n; i++)
		dst[i] = bf16_to_f32_host(tmp[i]);
	free(tmp);
	return 0;
}

/* ---- life cycle ------------------------------------------------------------------ */

extern "C" int64_t anni_lm_param_count(int d_model, int d_ff, int n_blocks, int vocab, int tied)
{
	int64_t D = d_model;
	int64_t FF = d_ff;
	int64_t V = vocab;
	int64_t n = D * V + V;

	if (!tied)
		n += V * D;
	n += (int64_t)n_blocks * (4 * D * D + D * FF + FF + FF * D + D + 4 * D);
	return n;
}

extern "C" anni_lm_adam *anni_lm_adam_create(const anni_lm_tensor *tensors, int n_tensors,
	int grad_dtype, int state_dtype)
{
	anni_lm_adam *opt;
	int64_t off = 0;
	int i;

	if (!tensors || n_tensors <= 0)
		return NULL;
	if ((grad_dtype != ANNI_DT_F32 && grad_dtype != ANNI_DT_BF16)
	    || (state_dtype != ANNI_DT_F32 && state_dtype != ANNI_DT_BF16))
		return NULL;
	opt = (anni_lm_adam *)calloc(1, sizeof(*opt));
	if (!opt)
		return NULL;
	opt->segs = (anni_lm_adam_seg *)calloc((size_t)n_tensors, sizeof(anni_lm_adam_seg));
	if (!opt->segs) {
		free(opt);
		return NULL;
	}
	for (i = 0; i < n_tensors; i++) {
		if (!tensors[i].w || tensors[i].n <= 0)
			continue;	/* the reference skips absent tensors too (lm_adam.c:30-31) */
		opt->segs[opt->n_segs].w = tensors[i].w;
		opt->segs[opt->n_segs].dw = tensors[i].dw;
		opt->segs[opt->n_segs].off = off;
		opt->segs[opt->n_segs].n = tensors[i].n;
		opt->segs[opt->n_segs].flags = tensors[i].flags;
		opt->n_segs++;
		off += tensors[i].n;
	}
	opt->n = off;
	opt->beta1 = 0.9;
	opt->beta2 = 0.999;
	opt->eps = 1e-8;
	opt->grad_dtype = grad_dtype;
	opt->state_dtype = state_dtype;
	/* the double-precision update term costs 4-6 % next to fp32 moments, ~14 % next to bf16 ones */
	opt->exact_update = state_dtype == ANNI_DT_F32;
	opt->h_m = (float *)calloc((size_t)(off > 0 ? off : 1), sizeof(float));
	opt->h_v = (float *)calloc((size_t)(off > 0 ? off : 1), sizeof(float));
	if (!opt->h_m || !opt->h_v || opt->n_segs == 0) {
		anni_lm_adam_free(&opt);
		return NULL;
	}
	return opt;
}

/*
** Nobody may keep a pointer into a flat that is about to go: matrix views set by
** anni_lm_adam_alias are detached (unalias_segs, lang/lm_adam.c:146-165 of the reference), and
** the gradient vectors registered by anni_lm_adam_alias_vec are forgotten.
*/
static void detach_views(anni_lm_adam *opt)
{
	for (int i = 0; i < opt->n_segs; i++) {
		anni_lm_adam_seg *s = &opt->segs[i];

		if (s->w_mat && opt->d_param && s->w_mat->d_data == opt->d_param + s->off) {
			s->w_mat->d_data = NULL;
			s->w_mat->on_device = 0;
		}
		if (s->dw_mat && opt->d_grad && s->dw_mat->d_data == (float *)opt->d_grad + s->off) {
			s->dw_mat->d_data = NULL;
			s->dw_mat->on_device = 0;
		}
		s->w_mat = s->dw_mat = NULL;
	}
	if (opt->d_grad)
		anni_colsum_forget(opt->d_grad, (char *)opt->d_grad + (size_t)opt->n * 4u);
}

static void release_device(anni_lm_adam *opt)
{
	detach_views(opt);
	if (opt->engine)
		anni_optstep_destroy(opt->engine);
	opt->engine = NULL;
	cudaFree(opt->d_param);
	cudaFree(opt->d_param_bf16);
	cudaFree(opt->d_param_fp8);
	if (opt->grad_arena_bytes)
		(void)anni_arena_free(opt->d_grad, opt->grad_arena_bytes);
	else
		cudaFree(opt->d_grad);
	opt->grad_arena_bytes = 0;
	cudaFree(opt->d_m);
	cudaFree(opt->d_v);
	opt->d_param = NULL;
	opt->d_param_bf16 = opt->d_param_fp8 = opt->d_grad = opt->d_m = opt->d_v = NULL;
	opt->dev_mv = 0;
	opt->params_valid = 0;
	gpu_adam_set_bf16_flat(NULL, NULL, 0);
}

extern "C" void anni_lm_adam_free(anni_lm_adam **popt)
{
	anni_lm_adam *opt;

	if (!popt || !*popt)
		return;
	opt = *popt;
	if (opt->d_param)
		(void)anni_lm_adam_sync_host(opt);	/* weights back to the host before the flats go (lm_adam.c:146-165) */
	if (opt->snap_stream) {
		cudaStreamSynchronize((cudaStream_t)opt->snap_stream);
		cudaEventDestroy((cudaEvent_t)opt->snap_event);
		cudaStreamDestroy((cudaStream_t)opt->snap_stream);
		cudaFreeHost(opt->snap_m);
		cudaFreeHost(opt->snap_v);
	}
	release_device(opt);
	free(opt->h_m);
	free(opt->h_v);
	free(opt->segs);
	free(opt);
	*popt = NULL;
}

extern "C" void anni_lm_adam_invalidate(anni_lm_adam *opt)
{
	if (opt)
		opt->params_valid = 0;
}

extern "C" void anni_lm_adam_set_offload(int on)
{
	g_offload_all = on ? 1 : 0;
}

extern "C" int anni_lm_adam_set_moments(anni_lm_adam *opt, const float *m, const float *v)
{
	if (!opt || !m || !v)
		return ANNI_E_ARG;
	memcpy(opt->h_m, m, (size_t)opt->n * sizeof(float));
	memcpy(opt->h_v, v, (size_t)opt->n * sizeof(float));
	opt->dev_mv = 0;
	if (opt->d_m) {		/* device copies are stale now: re-upload at the next step */
		cudaFree(opt->d_m);
		cudaFree(opt->d_v);
		opt->d_m = opt->d_v = NULL;
	}
	return ANNI_OK;
}

static int upload_weights(anni_lm_adam *opt)
{
	int i;

	for (i = 0; i < opt->n_segs; i++) {
		const anni_lm_adam_seg *s = &opt->segs[i];

		if (cudaMemcpy(opt->d_param + s->off, s->w, (size_t)s->n * 4u, cudaMemcpyHostToDevice)
		    != cudaSuccess)
			return -1;
	}
	/* one-shot fp32 -> bf16 of the whole flat, then publish it (lm_adam.c:284-290) */
	if (opt->n > 0x7fffffff) {
		/* the registry's int count cannot describe it; the twin is still seeded by the first step */
		gpu_adam_set_bf16_flat(NULL, NULL, 0);
	} else {
		if (gpu_adam_seed_bf16_flat(opt->d_param_bf16, opt->d_param, (int)opt->n) != 0)
			return -1;
		gpu_adam_set_bf16_flat(opt->d_param_bf16, opt->d_param, (int)opt->n);
	}
	gpu_device_sync();
	opt->params_valid = 1;
	gpu_half_wt_invalidate(NULL);
	return 0;
}

/* First use: the device flats, the engine and its tensor table (gpu_buffers_init, lm_adam.c:217-311). */
static int ensure_device(anni_lm_adam *opt)
{
	const size_t n = (size_t)opt->n;
	int any_fp8 = 0;
	int i;

	if (!gpu_available())
		return ANNI_E_CUDA;
	if (!opt->d_param) {
		anni_optstep_config cfg;
		int64_t *off;
		uint32_t *flg;

		for (i = 0; i < opt->n_segs; i++)
			if (opt->segs[i].flags & ANNI_SEG_TWIN_FP8)
				any_fp8 = 1;
		/*
		** The gradient flat goes into compressible memory where the device has it: every step
		** leaves it zeroed, and zero lines then cost a fraction of their size on the way to HBM
		** (about 4 % of the step at 555 M parameters).  Plain memory otherwise.
		*/
		if (anni_arena_alloc(n * elem_size(opt->grad_dtype), &opt->d_grad, &opt->grad_arena_bytes,
		    NULL) != ANNI_OK) {
			opt->d_grad = NULL;
			opt->grad_arena_bytes = 0;
			(void)cudaGetLastError();
		}
		if (cudaMalloc((void **)&opt->d_param, n * 4u) != cudaSuccess
		    || (!opt->d_grad && (cudaMalloc(&opt->d_grad, n * elem_size(opt->grad_dtype)) != cudaSuccess
		    || cudaMemset(opt->d_grad, 0, n * elem_size(opt->grad_dtype)) != cudaSuccess))
		    || cudaMalloc(&opt->d_param_bf16, n * 2u) != cudaSuccess
		    || (any_fp8 && cudaMalloc(&opt->d_param_fp8, n) != cudaSuccess)
		    || cudaMemset(opt->d_param_bf16, 0, n * 2u) != cudaSuccess
		    || (any_fp8 && cudaMemset(opt->d_param_fp8, 0, n) != cudaSuccess)) {
			(void)cudaGetLastError();
			release_device(opt);
			return ANNI_E_NOMEM;
		}
		off = (int64_t *)malloc((size_t)(opt->n_segs + 1) * sizeof(int64_t));
		flg = (uint32_t *)malloc((size_t)opt->n_segs * sizeof(uint32_t));
		if (!off || !flg) {
			free(off);
			free(flg);
			release_device(opt);
			return ANNI_E_NOMEM;
		}
		for (i = 0; i < opt->n_segs; i++) {
			off[i] = opt->segs[i].off;
			flg[i] = opt->segs[i].flags;
		}
		off[opt->n_segs] = opt->n;
		memset(&cfg, 0, sizeof(cfg));
		cfg.n_arena = (uint64_t)opt->n;
		cfg.shard_off = 0;
		cfg.shard_n = (uint64_t)opt->n;
		cfg.grad_dtype = opt->grad_dtype;
		cfg.state_dtype = opt->state_dtype;
		cfg.n_seg = opt->n_segs;
		cfg.seg_off = off;
		cfg.seg_flags = flg;
		i = anni_optstep_create(&cfg, &opt->engine);
		free(off);
		free(flg);
		if (i != ANNI_OK) {
			release_device(opt);
			return i;
		}
		opt->params_valid = 0;
	}
	if (!opt->params_valid && upload_weights(opt) != 0) {
		release_device(opt);
		return ANNI_E_CUDA;
	}
	if (!opt->d_m) {	/* first step, after set_moments, or after an offload */
		anni_optstep_buffers buf;

		if (cudaMalloc(&opt->d_m, n * elem_size(opt->state_dtype)) != cudaSuccess
		    || cudaMalloc(&opt->d_v, n * elem_size(opt->state_dtype)) != cudaSuccess) {
			(void)cudaGetLastError();
			cudaFree(opt->d_m);
			opt->d_m = opt->d_v = NULL;
			return ANNI_E_NOMEM;
		}
		if (upload_as(opt->d_m, opt->state_dtype, opt->h_m, opt->n) != 0
		    || upload_as(opt->d_v, opt->state_dtype, opt->h_v, opt->n) != 0) {
			/* half-filled flats must not pass for moments at the next call */
			cudaFree(opt->d_m);
			cudaFree(opt->d_v);
			opt->d_m = opt->d_v = NULL;
			return ANNI_E_CUDA;
		}
		buf.master = opt->d_param;
		buf.m = opt->d_m;
		buf.v = opt->d_v;
		buf.grad = opt->d_grad;
		buf.twin_bf16 = opt->d_param_bf16;
		buf.twin_fp8 = opt->d_param_fp8;
		i = anni_optstep_bind(opt->engine, &buf);
		if (i != ANNI_OK)
			return i;
	}
	if (g_offload_all)
		opt->offload_mv = 1;
	return ANNI_OK;
}

extern "C" int anni_lm_adam_prepare(anni_lm_adam *opt)
{
	return opt ? ensure_device(opt) : ANNI_E_ARG;
}

extern "C" int anni_lm_adam_alias(anni_lm_adam *opt, int tensor, anni_mat *w, anni_mat *dw)
{
	anni_lm_adam_seg *s;

	if (!opt || tensor < 0 || tensor >= opt->n_segs || !w || !opt->d_param)
		return ANNI_E_ARG;
	s = &opt->segs[tensor];
	if ((int64_t)w->rows * w->cols != s->n || (dw && (int64_t)dw->rows * dw->cols != s->n))
		return ANNI_E_ARG;
	if (dw && opt->grad_dtype != ANNI_DT_F32)
		return ANNI_E_ARG;	/* a float matrix cannot be a view of a bf16 flat */
	w->d_data = opt->d_param + s->off;
	w->on_device = 3;
	s->w_mat = w;
	if (dw) {
		dw->d_data = (float *)opt->d_grad + s->off;
		dw->on_device = 3;
		s->dw_mat = dw;
		s->dw = NULL;	/* gradients of this tensor now arrive on the device */
	}
	return ANNI_OK;
}

extern "C" int anni_lm_adam_alias_vec(anni_lm_adam *opt, int tensor, float **d_w, void **d_dw)
{
	anni_lm_adam_seg *s;
	void *grad_slice;

	if (!opt || tensor < 0 || tensor >= opt->n_segs || !opt->d_param || !opt->d_grad)
		return ANNI_E_ARG;
	s = &opt->segs[tensor];
	grad_slice = (char *)opt->d_grad + (size_t)s->off * elem_size(opt->grad_dtype);
	if (s->dw) {
		/* what the host vector holds so far goes over once; from now on the slice is the gradient */
		if (upload_as(grad_slice, opt->grad_dtype, s->dw, s->n) != 0)
			return ANNI_E_CUDA;
		if (opt->grad_dtype == ANNI_DT_F32 && s->n <= 0x7fffffff)
			(void)anni_colsum_register(s->dw, (float *)grad_slice, (int)s->n);
		s->dw = NULL;
	}
	if (d_w)
		*d_w = opt->d_param + s->off;
	if (d_dw)
		*d_dw = grad_slice;
	return ANNI_OK;
}

extern "C" int anni_lm_adam_snapshot_begin(anni_lm_adam *opt)
{
	const size_t nb = opt ? (size_t)opt->n * elem_size(opt->state_dtype) : 0;
	cudaStream_t st;
	cudaEvent_t ev;

	if (!opt || !opt->d_m || !opt->d_v)
		return ANNI_E_ARG;
	if (!opt->snap_stream) {
		st = NULL;
		ev = NULL;
		if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess
		    || cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess
		    || cudaMallocHost(&opt->snap_m, nb) != cudaSuccess
		    || cudaMallocHost(&opt->snap_v, nb) != cudaSuccess) {
			(void)cudaGetLastError();
			if (opt->snap_m)
				cudaFreeHost(opt->snap_m);
			opt->snap_m = opt->snap_v = NULL;	/* snap_v is the last to be set: never left allocated */
			if (ev)
				cudaEventDestroy(ev);
			if (st)
				cudaStreamDestroy(st);
			return ANNI_E_NOMEM;
		}
		opt->snap_stream = st;
		opt->snap_event = ev;
	}
	st = (cudaStream_t)opt->snap_stream;
	ev = (cudaEvent_t)opt->snap_event;
	/* the copies start once everything queued so far on the step stream (the legacy stream) is done */
	if (cudaEventRecord(ev, 0) != cudaSuccess || cudaStreamWaitEvent(st, ev, 0) != cudaSuccess
	    || cudaMemcpyAsync(opt->snap_m, opt->d_m, nb, cudaMemcpyDeviceToHost, st) != cudaSuccess
	    || cudaMemcpyAsync(opt->snap_v, opt->d_v, nb, cudaMemcpyDeviceToHost, st) != cudaSuccess)
		return ANNI_E_CUDA;
	return ANNI_OK;
}

extern "C" int anni_lm_adam_snapshot_finish(anni_lm_adam *opt)
{
	int64_t i;

	if (!opt || !opt->snap_stream)
		return ANNI_E_ARG;
	if (cudaStreamSynchronize((cudaStream_t)opt->snap_stream) != cudaSuccess)
		return ANNI_E_CUDA;
	if (opt->state_dtype == ANNI_DT_F32) {
		memcpy(opt->h_m, opt->snap_m, (size_t)opt->n * 4u);
		memcpy(opt->h_v, opt->snap_v, (size_t)opt->n * 4u);
	} else {
		const uint16_t *pm = (const uint16_t *)opt->snap_m;
		const uint16_t *pv = (const uint16_t *)opt->snap_v;

		for (i = 0; i < opt->n; i++) {
			opt->h_m[i] = bf16_to_f32_host(pm[i]);
			opt->h_v[i] = bf16_to_f32_host(pv[i]);
		}
	}
	return ANNI_OK;
}

extern "C" int anni_lm_adam_upload_grads(anni_lm_adam *opt)
{
	int i;

	if (!opt || !opt->d_grad)
		return ANNI_E_ARG;
	for (i = 0; i < opt->n_segs; i++) {
		const anni_lm_adam_seg *s = &opt->segs[i];

		if (!s->dw)
			continue;
		if (upload_as((char *)opt->d_grad + (size_t)s->off * elem_size(opt->grad_dtype),
		    opt->grad_dtype, s->dw, s->n) != 0)
			return ANNI_E_CUDA;
	}
	return ANNI_OK;
}

extern "C" void anni_lm_adam_zero_grad(anni_lm_adam *opt)
{
	int i;

	if (!opt)
		return;
	for (i = 0; i < opt->n_segs; i++)
		if (opt->segs[i].dw)
			memset(opt->segs[i].dw, 0, (size_t)opt->segs[i].n * sizeof(float));
	if (opt->d_grad)
		(void)cudaMemset(opt->d_grad, 0, (size_t)opt->n * elem_size(opt->grad_dtype));
}

extern "C" int anni_lm_adam_sync_host(anni_lm_adam *opt)
{
	int i;

	if (!opt)
		return ANNI_E_ARG;
	if (opt->d_param && opt->params_valid) {
		if (cudaDeviceSynchronize() != cudaSuccess)
			return ANNI_E_CUDA;
		for (i = 0; i < opt->n_segs; i++) {
			const anni_lm_adam_seg *s = &opt->segs[i];

			if (cudaMemcpy(s->w, opt->d_param + s->off, (size_t)s->n * 4u,
			    cudaMemcpyDeviceToHost) != cudaSuccess)
				return ANNI_E_CUDA;
		}
	}
	if (!opt->dev_mv || !opt->d_m || !opt->d_v)
		return ANNI_OK;
	if (download_as(opt->h_m, opt->d_m, opt->state_dtype, opt->n) != 0
	    || download_as(opt->h_v, opt->d_v, opt->state_dtype, opt->n) != 0)
		return ANNI_E_CUDA;
	opt->dev_mv = 0;
	return ANNI_OK;
}

/* ---- the step ----------------------------------------------------------------------- */

/*
** Uploads the host gradient arrays and clears them (seg_gather / seg_scatter, lm_adam.c:361-413
** of the reference).  With a model's worth of them (hundreds of megabytes when every gradient
** lives on the host) one core needs tens of milliseconds for the clearing alone, so the arrays
** are cut into pieces of at most 1 Mi elements, dealt out to a few threads, and a piece is
** cleared as soon as ITS upload is through, beside the uploads of the later ones: the step then
** costs the longer of the two instead of their sum, and what is left after the last upload is
** one piece per thread.  Pinned fp32 gradients go up with asynchronous copies, back to back on
** the default stream, an event behind each piece telling the threads when its source may
** change; anything else with blocking copies.  Small totals are cleared in place after the
** launch.
*/
struct grad_clearer {
	struct piece {
		float	*src;
		int64_t	n;
		int64_t	off;	/* element offset in the gradient flat */
	};
	static const int64_t	PIECE = (int64_t)1 << 20;

	anni_lm_adam		*opt = nullptr;
	std::vector<piece>	pieces;
	std::vector<cudaEvent_t> ev;		/* async: one per piece */
	std::atomic<int>	ready{0};	/* pieces [0, ready) have been handed to the copy */
	std::atomic<int>	stop{0};
	std::thread		th[16];
	int			n_th = 0;
	bool			async = false;
	int			device = 0;

	static bool pinned(const void *p)
	{
		cudaPointerAttributes at;

		if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
			(void)cudaGetLastError();
			return false;
		}
		return at.type == cudaMemoryTypeHost;
	}
	void start(anni_lm_adam *o)
	{
		const unsigned hw = std::thread::hardware_concurrency();
		int64_t total = 0;

		opt = o;
		for (int i = 0; i < o->n_segs; i++) {
			const anni_lm_adam_seg *sg = &o->segs[i];

			if (!sg->dw)
				continue;
			total += sg->n;
			for (int64_t at = 0; at < sg->n; at += PIECE)
				pieces.push_back({ sg->dw + at, sg->n - at < PIECE ? sg->n - at : PIECE, sg->off + at });
		}
		if (total < ((int64_t)32 << 20))
			return;			/* cleared by finish() after the launch */
		n_th = hw >= 16 ? 12 : hw >= 8 ? 6 : 2;	/* the caller's own thread only queues copies and waits */
		async = o->grad_dtype == ANNI_DT_F32 && cudaGetDevice(&device) == cudaSuccess;
		for (int i = 0; async && i < o->n_segs; i++)
			if (o->segs[i].dw && o->segs[i].n > 0 && !pinned(o->segs[i].dw))
				async = false;
		if (async) {
			ev.assign(pieces.size(), nullptr);
			for (size_t k = 0; k < pieces.size(); k++)
				if (cudaEventCreateWithFlags(&ev[k], cudaEventDisableTiming) != cudaSuccess) {
					ev[k] = nullptr;
					async = false;	/* the events made so far go with the object */
					break;
				}
		}
		for (int k = 0; k < n_th; k++)
			th[k] = std::thread([this, k]() {
				if (async)
					(void)cudaSetDevice(device);
				for (size_t i = (size_t)k; i < pieces.size(); i += (size_t)n_th) {
					while (ready.load(std::memory_order_acquire) <= (int)i) {
						if (stop.load(std::memory_order_relaxed))
							return;
						std::this_thread::yield();
					}
					if (async && cudaEventSynchronize(ev[i]) != cudaSuccess)
						return;		/* the step reports the error; the gradients stay */
					memset(pieces[i].src, 0, (size_t)pieces[i].n * sizeof(float));
				}
			});
	}
	/* every piece to the device, in order; 0 or -1 */
	int upload_all()
	{
		const size_t esz = elem_size(opt->grad_dtype);

		for (size_t i = 0; i < pieces.size(); i++) {
			const piece &pc = pieces[i];
			void *dst = (char *)opt->d_grad + (size_t)pc.off * esz;

			if (!async) {
				if (upload_as(dst, opt->grad_dtype, pc.src, pc.n) != 0)
					return -1;
			} else if (cudaMemcpyAsync(dst, pc.src, (size_t)pc.n * sizeof(float), cudaMemcpyHostToDevice, 0)
			    != cudaSuccess || cudaEventRecord(ev[i], 0) != cudaSuccess)
				return -1;
			ready.store((int)i + 1, std::memory_order_release);
		}
		return 0;
	}
	/* after the launch: waits for the threads, or clears small totals here */
	void finish()
	{
		if (!opt)
			return;
		if (n_th == 0)
			for (const piece &pc : pieces)
				memset(pc.src, 0, (size_t)pc.n * sizeof(float));
		join();
		opt = nullptr;
	}
	void join()
	{
		for (int k = 0; k < n_th; k++)
			if (th[k].joinable())
				th[k].join();
		n_th = 0;
	}
	~grad_clearer()		/* a step that failed on the way: what was not uploaded stays as it is */
	{
		stop.store(1, std::memory_order_relaxed);
		join();
		for (cudaEvent_t e : ev)
			if (e)
				(void)cudaEventDestroy(e);
	}
};

static double now_us(void)
{
	return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

static int step_trace(void)
{
	static int on = -1;

	if (on < 0) {
		const char *e = getenv("ANNI_B200_STEP_TRACE");

		on = e && atoi(e) != 0;
	}
	return on;
}

/* ANN_GNORM_EVERY=k: report the gradient norm every k-th step (adam_gnorm_every, lm_adam.c:438-450) */
static int gnorm_every(void)
{
	static int every = -1;

	if (every < 0) {
		const char *e = getenv("ANN_GNORM_EVERY");

		every = e ? atoi(e) : 0;
		if (every < 0)
			every = 0;
	}
	return every;
}

extern "C" int anni_lm_adam_step(anni_lm_adam *opt, double lr)
{
	return anni_lm_adam_step_scaled(opt, lr, 1.0);
}

extern "C" int anni_lm_adam_step_scaled(anni_lm_adam *opt, double lr, double grad_scale)
{
	anni_optstep_hyper hp;
	anni_optstep_status st;
	grad_clearer clearer;
	double t_mark[5] = { now_us(), 0.0, 0.0, 0.0, 0.0 };
	int host_grads = 0;
	int rc;
	int i;

	if (!opt || !(lr > 0.0))
		return ANNI_OK;		/* lm_adam.c:531: nothing happens, t unchanged */
	opt->t++;			/* before anything can skip or fail (lm_adam.c:533) */
	opt->last_error = 0;
	rc = ensure_device(opt);
	if (rc != ANNI_OK)
		goto fail;
	for (i = 0; i < opt->n_segs; i++)
		if (opt->segs[i].dw)
			host_grads = 1;
	t_mark[1] = now_us();
	if (host_grads) {		/* seg_gather (lm_adam.c:361-396) for host-resident gradients */
		if (!opt->d_grad) {
			rc = ANNI_E_ARG;
			goto fail;
		}
		clearer.start(opt);
		t_mark[1] = now_us();
		if (clearer.upload_all() != 0) {
			rc = ANNI_E_CUDA;
			goto fail;
		}
	}
	t_mark[2] = now_us();
	memset(&hp, 0, sizeof(hp));
	hp.lr = lr;
	hp.beta1 = opt->beta1;
	hp.beta2 = opt->beta2;
	hp.eps = opt->eps;
	hp.weight_decay = opt->weight_decay;
	hp.grad_clip = opt->grad_clip;
	hp.grad_scale = opt->loss_scale > 0.0 ? grad_scale / opt->loss_scale : grad_scale;
	hp.t = opt->t;
	hp.flags = ANNI_STEP_ZERO_GRAD;
	if (opt->exact_update)
		hp.flags |= ANNI_STEP_EXACT_UPDATE;
	/* the reference computes the norm (and may skip) only when it clips or reports it (lm_adam.c:466) */
	if (opt->grad_clip > 0.0 || opt->loss_scale > 0.0 || gnorm_every() > 0)
		hp.flags |= ANNI_STEP_CHECK_FINITE;
	rc = anni_optstep_step(opt->engine, &hp, NULL);
	if (rc != ANNI_OK)
		goto fail;
	t_mark[3] = now_us();
	clearer.finish();		/* the host gradient vectors are zero from here on (lm_adam.c:413) */
	t_mark[4] = now_us();
	rc = anni_optstep_status_read(opt->engine, &st, NULL);
	if (step_trace())		/* ANNI_B200_STEP_TRACE=1: where the host side of a step spends its time */
		fprintf(stderr, "[adam] step %d host us: prepare %.0f, uploads queued %.0f, launch %.0f, "
		    "clearing waited %.0f, status %.0f\n", opt->t, t_mark[1] - t_mark[0], t_mark[2] - t_mark[1],
		    t_mark[3] - t_mark[2], t_mark[4] - t_mark[3], now_us() - t_mark[4]);
	if (rc == ANNI_OK && st.error != 0)
		rc = st.error;
	if (rc != ANNI_OK)
		goto fail;
	if (hp.flags & ANNI_STEP_CHECK_FINITE)
		opt->last_grad_norm = st.norm;
	opt->last_skipped = st.skipped;
	if (st.skipped)
		fprintf(stderr, "[adam] step %d skipped: grad norm %g\n", opt->t, st.norm);
	else {
		opt->dev_mv = 1;
		if (gnorm_every() > 0 && opt->t % gnorm_every() == 0)	/* lm_adam.c:484-487 */
			fprintf(stderr, "[adam] step %d grad norm %.4g%s\n", opt->t, st.norm,
			    opt->grad_clip > 0.0 && st.norm > opt->grad_clip ? " (clipped)" : "");
	}
	opt->params_valid = 1;
	gpu_half_wt_invalidate(NULL);	/* lm_adam.c:547: derived copies rebuild */
	if (opt->offload_mv) {		/* adam_offload_mv (lm_adam.c:314-334) */
		if (download_as(opt->h_m, opt->d_m, opt->state_dtype, opt->n) == 0
		    && download_as(opt->h_v, opt->d_v, opt->state_dtype, opt->n) == 0) {
			cudaFree(opt->d_m);
			cudaFree(opt->d_v);
			opt->d_m = opt->d_v = NULL;
			opt->dev_mv = 0;
		}
	}
	return ANNI_OK;
fail:
	/* params_valid stays as it is: a step refused for its arguments leaves the device weights the
	** newest copy, and re-reading the host arrays would lose the steps taken so far */
	opt->last_error = rc;
	fprintf(stderr, "[adam] step %d: device step failed (%d); no host fallback in this library\n",
	    opt->t, rc);
	return rc;
}

/* ---- gradient-buffer helpers (lang/gradutil.c of the reference) ---------------------------- */

static size_t mat_bytes(const anni_mat *m)
{
	return (size_t)m->rows * (size_t)m->cols * sizeof(float);
}

/* mat_zero (gradutil.c:8-22): zero whichever side is authoritative. */
extern "C" void anni_mat_zero(anni_mat *m)
{
	if (!m)
		return;
	if (m->d_data && m->on_device != 0 && gpu_available() && gpu_memset(m->d_data, 0, mat_bytes(m)) == 0) {
		if (m->on_device != 3)
			m->on_device = 1;	/* device-authoritative; an aliased view stays aliased */
		return;
	}
	if (!m->data)
		return;
	memset(m->data, 0, mat_bytes(m));
	m->on_device = 0;
}

/* mat_zero_dev (gradutil.c:29-50): zero host and device twin together; an aliased view stays aliased. */
extern "C" void anni_mat_zero_dev(anni_mat *m)
{
	if (!m)
		return;
	if (m->d_data && gpu_available() && gpu_memset(m->d_data, 0, mat_bytes(m)) == 0) {
		if (m->on_device == 3)
			return;
		if (m->data) {
			memset(m->data, 0, mat_bytes(m));
			m->on_device = 2;
		} else
			m->on_device = 1;
		return;
	}
	if (!m->data)
		return;
	memset(m->data, 0, mat_bytes(m));
	m->on_device = 0;
}

/* vec_zero (gradutil.c:52-56). */
extern "C" void anni_vec_zero(anni_vec *v)
{
	if (v && v->data)
		memset(v->data, 0, (size_t)v->n * sizeof(float));
}

/* mat_axpy (gradutil.c:58-75), device part only: 0 when y += a x ran on the GPU, else ANNI_E_*. */
extern "C" int anni_mat_axpy(anni_mat *y, double a, const anni_mat *x)
{
	if (!y || !x || y->rows != x->rows || y->cols != x->cols)
		return ANNI_E_ARG;
	return gpu_mat_axpy(y, a, x) == 0 ? ANNI_OK : ANNI_E_CUDA;
}

/* ---- LR schedule ---------------------------------------------------------------------- */

extern "C" double anni_lr_schedule(double base_lr, int step, int warmup_steps, int decay_steps,
	const char *decay_kind, int sched_from)
{
	double frac;
	int past;

	step -= sched_from;
	if (step < 0)
		step = 0;
	if (warmup_steps > 0 && step < warmup_steps)
		return base_lr * ((double)step + 1.0) / (double)warmup_steps;
	if (decay_steps <= 0 || !decay_kind || strcmp(decay_kind, "none") == 0)
		return base_lr;
	past = step - warmup_steps;
	if (past < 0)
		past = 0;
	if (past > decay_steps)
		past = decay_steps;
	frac = (double)past / (double)decay_steps;
	if (strcmp(decay_kind, "linear") == 0)
		return base_lr * (1.0 - frac);
	return base_lr * 0.5 * (1.0 + cos(3.14159265358979323846 * frac));
}

/* ---- checkpoint: the Adam section --------------------------------------------------------- */

#define CKPT_PAIRS_PER_WRITE	(1 << 21)	/* 16 MB of (m, v) pairs per fwrite, as lm_serialize.c:261 */

static int write_adam_section(FILE *fp, int epoch, int step, int t, int64_t n, const float *m,
	const float *v)
{
	int32_t hdr[5];
	float *buf;
	int64_t i;
	int64_t k;
	int64_t cnt;

	if (n < 0 || n > 0x7fffffff)
		return -1;	/* the format stores n as int32 */
	hdr[0] = 1;
	hdr[1] = epoch;
	hdr[2] = step;
	hdr[3] = t;
	hdr[4] = (int32_t)n;
	if (fwrite(hdr, sizeof(int32_t), 5, fp) != 5)
		return -1;
	buf = (float *)malloc((size_t)CKPT_PAIRS_PER_WRITE * 2u * sizeof(float));
	if (!buf)
		return -1;
	for (i = 0; i < n; i += cnt) {
		cnt = n - i < CKPT_PAIRS_PER_WRITE ? n - i : CKPT_PAIRS_PER_WRITE;
		for (k = 0; k < cnt; k++) {
			buf[2 * k] = m[i + k];
			buf[2 * k + 1] = v[i + k];
		}
		if (fwrite(buf, sizeof(float), (size_t)cnt * 2u, fp) != (size_t)cnt * 2u) {
			free(buf);
			return -1;
		}
	}
	free(buf);
	return 0;
}

extern "C" int anni_ckpt_write_adam(const char *path, int append, int epoch, int step, int t,
	int64_t n, const float *m, const float *v)
{
	char tmp[1024];
	FILE *fp;
	int bad;

	if (!path || !m || !v)
		return ANNI_E_ARG;
	if (append) {
		fp = fopen(path, "ab");
		if (!fp)
			return ANNI_E_ARG;
		bad = write_adam_section(fp, epoch, step, t, n, m, v) != 0;
		if (fclose(fp) != 0)
			bad = 1;
		return bad ? ANNI_E_ARG : ANNI_OK;
	}
	/* whole file: write beside it and rename, so a crash keeps the previous checkpoint */
	if (snprintf(tmp, sizeof(tmp), "%s.tmp", path) >= (int)sizeof(tmp))
		return ANNI_E_ARG;
	fp = fopen(tmp, "wb");
	if (!fp)
		return ANNI_E_ARG;
	bad = write_adam_section(fp, epoch, step, t, n, m, v) != 0;
	if (fclose(fp) != 0)
		bad = 1;
	if (bad || rename(tmp, path) != 0) {
		remove(tmp);
		return ANNI_E_ARG;
	}
	return ANNI_OK;
}

extern "C" int anni_ckpt_read_adam(const char *path, int64_t offset, int64_t n_expected, int *epoch,
	int *step, int *t, float *m, float *v)
{
	FILE *fp;
	int32_t hdr[5];
	float *buf;
	int64_t i;
	int64_t k;
	int64_t cnt;
	long size;

	if (!path || n_expected < 0 || !m || !v)
		return ANNI_E_ARG;
	fp = fopen(path, "rb");
	if (!fp)
		return ANNI_E_ARG;
	if (offset < 0) {
		if (fseek(fp, 0, SEEK_END) != 0 || (size = ftell(fp)) < 0
		    || (int64_t)size < 20 + 8 * n_expected) {
			fclose(fp);
			return ANNI_E_ARG;
		}
		offset = (int64_t)size - (20 + 8 * n_expected);
	}
	/* the loader of the reference insists on has_adam == 1 and on the slot count (lm_serialize.c:549-562) */
	if (fseek(fp, (long)offset, SEEK_SET) != 0 || fread(hdr, sizeof(int32_t), 5, fp) != 5
	    || hdr[0] != 1 || (int64_t)hdr[4] != n_expected) {
		fclose(fp);
		return ANNI_E_ARG;
	}
	if (epoch)
		*epoch = hdr[1];
	if (step)
		*step = hdr[2];
	if (t)
		*t = hdr[3];
	buf = (float *)malloc((size_t)CKPT_PAIRS_PER_WRITE * 2u * sizeof(float));
	if (!buf) {
		fclose(fp);
		return ANNI_E_NOMEM;
	}
	for (i = 0; i < n_expected; i += cnt) {
		cnt = n_expected - i < CKPT_PAIRS_PER_WRITE ? n_expected - i : CKPT_PAIRS_PER_WRITE;
		if (fread(buf, sizeof(float), (size_t)cnt * 2u, fp) != (size_t)cnt * 2u) {
			free(buf);
			fclose(fp);
			return ANNI_E_ARG;
		}
		for (k = 0; k < cnt; k++) {
			m[i + k] = buf[2 * k];
			v[i + k] = buf[2 * k + 1];
		}
	}
	free(buf);
	fclose(fp);
	return ANNI_OK;
}
