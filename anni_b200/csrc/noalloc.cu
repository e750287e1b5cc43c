/*
** anni_optstep_step_noalloc: the fused step for callers that must not allocate.
**
** Who needs it: a trainer that has handed the whole device to its own arena
** allocator (so a later cudaMalloc can fail or fragment it), code that runs
** inside a region where the CUDA allocator may not be entered (a callback, a
** real-time loop, a process that forbids driver allocations after start-up),
** or a host that simply wants one self-contained call without creating an
** engine first.  The regular path keeps its working memory (barrier and
** ticket counters, per-block partial sums, the device copy of the tensor
** table, per-tensor amax and scale) in a block that anni_optstep_create
** allocates with cudaMalloc.  Here the same working memory is a fixed array
** inside the library image: it exists on every GPU that loads the library,
** for as long as the process lives, whether or not this call is ever used.
**
** Consequences the caller has to know:
**   - the tensor table is limited to ANNI_NOALLOC_MAX_SEG entries (the array
**     cannot grow); a longer table is refused with ANNI_E_LIMIT and nothing runs;
**   - every call on a device shares the one array.  It still holds what the
**     previous call left, so each call clears the counters, the error word and
**     the amax slots it is about to use before the step kernel starts.  Two
**     calls that overlap on the same GPU (different streams, or different host
**     threads) would trample each other's counters and partial sums: issue
**     them one after the other on one stream, or serialise them yourself;
**   - the first call on each device looks up the device address of the array
**     (and sizes the launch).  Make that first call during start-up, before any
**     stream capture is begun on that device;
**   - the dynamic loss-scale state machine lives in an engine's own block and is
**     not available here: pass the loss scale folded into grad_scale;
**   - cfg->seg_off and cfg->seg_flags are read from host memory during the call
**     (they must stay valid until it returns, not longer), and a stream that is
**     being captured is refused with ANNI_E_ARG.
** No cudaMalloc, cudaFree, or other allocating routine is called on any path
** below; the caller supplies every input and output buffer.
*/
#include <cuda_runtime.h>
#include <stddef.h>
#include <string.h>
#include <mutex>
#include "anni_b200.h"
#include "optstep_internal.h"

#define NOALLOC_MAX_DEVICES	64

struct noalloc_scratch {
	anni_control	ctl;
	int64_t		seg_off[ANNI_NOALLOC_MAX_SEG + 1];
	uint32_t	seg_flags[ANNI_NOALLOC_MAX_SEG];
	float		seg_amax[ANNI_NOALLOC_MAX_SEG];
	float		seg_scale[ANNI_NOALLOC_MAX_SEG];
	uint32_t	seg_done[ANNI_NOALLOC_MAX_SEG];	/* per-tensor arrival counters (fp8 twins) */
};

/*
** The working memory itself.  In host code this name is only a handle for
** cudaGetSymbolAddress; it is NOT a device pointer and must never be handed to
** a kernel as one.
*/
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(noalloc_scratch)];

/* Clears what has to start at zero; names the array directly, as device code may. */
__global__ void noalloc_clear_kernel(int n_seg)
{
	noalloc_scratch *s = reinterpret_cast<noalloc_scratch *>(g_noalloc_scratch);
	const int i = blockIdx.x * blockDim.x + threadIdx.x;

	if (i == 0) {
		s->ctl.reduce[0] = 0.0;
		s->ctl.reduce[1] = 0.0;
		s->ctl.norm = 0.0;
		s->ctl.eff_scale = 0.0;
		s->ctl.loss_scale = 0.0;	/* state machine off */
		s->ctl.good_steps = 0;
		s->ctl.skipped = 0;
		s->ctl.error = 0;
		s->ctl.bar_count = 0;
		s->ctl.norm_ticket = 0;
		s->ctl.done_ticket = 0;
	}
	if (i < n_seg) {
		s->seg_amax[i] = 0.0f;
		s->seg_scale[i] = 0.0f;
		s->seg_done[i] = 0u;
	}
}

namespace {

struct per_device {
	noalloc_scratch	*ptr;		/* device address of g_noalloc_scratch on this device */
	int		blocks[2][2];	/* persistent grid per (grad dtype, state dtype) */
	int		sc_log2;	/* super-chunk size, as the engines use it */
	bool		ready;
};

per_device g_dev[NOALLOC_MAX_DEVICES];
std::mutex g_dev_lock;

/* Once per device, with that device current: resolve the array's device address. */
int device_setup(int dev, per_device **out)
{
	std::lock_guard<std::mutex> hold(g_dev_lock);
	per_device *d;

	if (dev < 0 || dev >= NOALLOC_MAX_DEVICES)
		return ANNI_E_LIMIT;
	d = &g_dev[dev];
	if (!d->ready) {
		void *p = NULL;

		if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == NULL)
			return ANNI_E_CUDA;
		for (int g = 0; g < 2; g++)
			for (int s = 0; s < 2; s++) {
				/* the engines' own geometry: same grid, same block partials, same norm bits */
				if (anni_engine_geometry(g, s, &d->blocks[g][s], &d->sc_log2) != ANNI_OK)
					return ANNI_E_CUDA;
			}
		d->ptr = static_cast<noalloc_scratch *>(p);
		d->ready = true;
	}
	*out = d;
	return ANNI_OK;
}

}	/* namespace */

extern "C" int anni_optstep_step_noalloc(const anni_optstep_config *cfg,
	const anni_optstep_buffers *buf, const anni_optstep_hyper *hp, float *seg_scale_out,
	void *stream)
{
	cudaStream_t st = (cudaStream_t)stream;
	per_device *d = NULL;
	anni_launch la;
	int64_t one_off[2];
	uint32_t one_flag = ANNI_SEG_WD | ANNI_SEG_TWIN_BF16;
	const int64_t *off;
	const uint32_t *flg;
	uintptr_t bits;
	int n_seg;
	int has_fp8 = 0;
	int dev = -1;
	int rc;

	if (!cfg || !buf || !hp)
		return ANNI_E_ARG;
	if (cfg->n_seg > ANNI_NOALLOC_MAX_SEG)
		return ANNI_E_LIMIT;		/* the built-in table holds ANNI_NOALLOC_MAX_SEG tensors */
	if (cfg->n_seg < 0 || (cfg->n_seg > 0 && (!cfg->seg_off || !cfg->seg_flags)))
		return ANNI_E_ARG;
	if (cfg->shard_off > cfg->n_arena || cfg->shard_n > cfg->n_arena - cfg->shard_off)
		return ANNI_E_ARG;
	if ((cfg->grad_dtype != ANNI_DT_F32 && cfg->grad_dtype != ANNI_DT_BF16)
	    || (cfg->state_dtype != ANNI_DT_F32 && cfg->state_dtype != ANNI_DT_BF16))
		return ANNI_E_ARG;
	if (cfg->shard_n > 0 && (!buf->master || !buf->m || !buf->v || !buf->grad))
		return ANNI_E_ARG;
	if (hp->flags & ANNI_STEP_DEV_LOSS_SCALE)
		return ANNI_E_ARG;
	if (cfg->n_seg > 0) {
		n_seg = cfg->n_seg;
		off = cfg->seg_off;
		flg = cfg->seg_flags;
		if (off[0] != 0 || (uint64_t)off[n_seg] != cfg->n_arena)
			return ANNI_E_ARG;
		for (int i = 0; i < n_seg; i++) {
			if (off[i + 1] < off[i])
				return ANNI_E_ARG;
			if (flg[i] & ANNI_SEG_TWIN_FP8)
				has_fp8 = 1;
		}
	} else {
		n_seg = 1;
		one_off[0] = 0;
		one_off[1] = (int64_t)cfg->n_arena;
		off = one_off;
		flg = &one_flag;
	}
	if (has_fp8 && cfg->shard_n > 0 && !buf->twin_fp8)
		return ANNI_E_ARG;
	if (cudaGetDevice(&dev) != cudaSuccess)
		return ANNI_E_CUDA;
	{
		/* the tensor table travels from the caller's host memory with every call: a captured
		** copy would replay from an address that may be gone, so a capturing stream is refused */
		cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;

		if (cudaStreamIsCapturing(st, &cap) != cudaSuccess)
			return ANNI_E_CUDA;
		if (cap != cudaStreamCaptureStatusNone)
			return ANNI_E_ARG;
	}
	rc = device_setup(dev, &d);
	if (rc != ANNI_OK)
		return rc;

	memset(&la, 0, sizeof(la));
	la.master = buf->master;
	la.m = buf->m;
	la.v = buf->v;
	la.grad = buf->grad;
	la.twin16 = (uint16_t *)buf->twin_bf16;
	la.twin8 = (uint8_t *)buf->twin_fp8;
	bits = (uintptr_t)buf->master | (uintptr_t)buf->m | (uintptr_t)buf->v | (uintptr_t)buf->grad
	    | (uintptr_t)buf->twin_bf16 | (uintptr_t)buf->twin_fp8;
	la.aligned = (bits & 15) == 0;
	la.n = cfg->shard_n;
	la.arena_off = cfg->shard_off;
	la.seg_off = d->ptr->seg_off;
	la.seg_flags = d->ptr->seg_flags;
	la.seg_amax = d->ptr->seg_amax;
	la.seg_scale = d->ptr->seg_scale;
	la.seg_done = d->ptr->seg_done;
	la.n_seg = n_seg;
	la.sc_log2 = d->sc_log2;
	la.pipe_lag = ANNI_PIPE_LAG;
	la.ctl = &d->ptr->ctl;
	la.flags = has_fp8 ? ANNI_LAUNCH_HAS_FP8 : 0;
	rc = anni_fill_hyper(&la, hp);
	if (rc != ANNI_OK)
		return rc;

	/* the array keeps the previous call's contents: clear, then load this call's table */
	noalloc_clear_kernel<<<(n_seg + 255) / 256, 256, 0, st>>>(n_seg);
	anni_count_launch();
	if (cudaGetLastError() != cudaSuccess
	    || cudaMemcpyAsync(d->ptr->seg_off, off, (size_t)(n_seg + 1) * sizeof(int64_t),
	    cudaMemcpyHostToDevice, st) != cudaSuccess
	    || cudaMemcpyAsync(d->ptr->seg_flags, flg, (size_t)n_seg * sizeof(uint32_t),
	    cudaMemcpyHostToDevice, st) != cudaSuccess)
		return ANNI_E_CUDA;
	rc = anni_launch_fused(&la, cfg->grad_dtype, cfg->state_dtype,
	    d->blocks[cfg->grad_dtype][cfg->state_dtype], st);
	if (rc != ANNI_OK)
		return rc;
	if (seg_scale_out && has_fp8
	    && cudaMemcpyAsync(seg_scale_out, d->ptr->seg_scale, (size_t)n_seg * sizeof(float),
	    cudaMemcpyDeviceToDevice, st) != cudaSuccess)
		return ANNI_E_CUDA;
	return ANNI_OK;
}

extern "C" int anni_optstep_status_noalloc(anni_optstep_status *out, void *stream)
{
	per_device *d = NULL;
	anni_control head;
	int dev = -1;
	int rc;

	if (!out)
		return ANNI_E_ARG;
	if (cudaGetDevice(&dev) != cudaSuccess)
		return ANNI_E_CUDA;
	rc = device_setup(dev, &d);
	if (rc != ANNI_OK)
		return rc;
	if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess
	    || cudaMemcpy(&head, &d->ptr->ctl, offsetof(anni_control, partials),
	    cudaMemcpyDeviceToHost) != cudaSuccess)
		return ANNI_E_CUDA;
	out->sumsq = head.reduce[0];
	out->norm = head.norm;
	out->eff_scale = head.eff_scale;
	out->loss_scale = 0.0;
	out->skipped = head.skipped;
	out->error = head.error;
	out->good_steps = 0;
	out->steps_done = head.steps_done;
	return ANNI_OK;
}
