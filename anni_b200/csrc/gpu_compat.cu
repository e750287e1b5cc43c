/*
** The reference trainer's device API (num/gpu.h of the reference project) on
** top of this library's kernels, so that the trainer links libanni_b200.so in
** place of its own CUDA object.  Two parts:
**
**  - real bodies for what the optimizer path calls (memory, stream, the flat
**    bf16 twin registry, gpu_grad_sumsq, gpu_adam_step_dev_bf16, gpu_mat_axpy);
**  - "not on the device" answers for everything else, with the return values the
**    reference's stub backend gives (num/gpu_stub.c), which its callers treat
**    as "use the CPU path".
**
** All work is queued on one process-wide blocking stream, as the reference
** does (num/gpu_cuda.cu:37-44): the optimizer is called from the single
** training thread.  Errors are never fatal: -1 / NULL, and the pending CUDA
** error can be polled with gpu_debug_last_error().
*/
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <mutex>
#include <unordered_map>
#include "anni_gpu_compat.h"
#include "optstep_internal.h"

namespace {

std::once_flag g_once;
int g_have_gpu;
cudaStream_t g_st;
int g_sync_mode_v;
int g_prec = ANNI_GPU_PREC_FP32;
int g_fp8_on;
int g_fp8_dgrad_on;
double g_adam_wd;
unsigned g_wt_epoch;
void *g_flat_bf16;
const float *g_flat_fp32;
size_t g_flat_n;
std::mutex g_malloc_lock;	/* gpu_malloc may be entered from worker threads (gpu_cuda.cu:2644) */
std::unordered_map<void *, size_t> g_arena_blocks;	/* blocks handed out by anni_arena_alloc -> mapped size */

/* device state of the two legacy optimizer calls, created on first use */
struct legacy_state {
	anni_control	*ctl;
	int64_t		*seg_off;	/* {0, 2^62}: one tensor covering any n */
	uint32_t	*flags_twin;	/* decay + bf16 twin */
	uint32_t	*flags_plain;	/* decay only */
	float		*amax;
	int		blocks;
} g_legacy;

void init_once(void)
{
	int n = 0;

	if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
		(void)cudaGetLastError();
		g_have_gpu = 0;
		return;
	}
	if (cudaStreamCreate(&g_st) != cudaSuccess) {
		g_have_gpu = 0;
		return;
	}
	g_have_gpu = 1;
}

int legacy_ready(void)
{
	static const int64_t off[2] = { 0, (int64_t)1 << 62 };
	static const uint32_t f_twin = ANNI_SEG_WD | ANNI_SEG_TWIN_BF16;
	static const uint32_t f_plain = ANNI_SEG_WD;

	if (g_legacy.ctl)
		return 0;
	if (cudaMalloc((void **)&g_legacy.ctl, sizeof(anni_control)) != cudaSuccess
	    || cudaMalloc((void **)&g_legacy.seg_off, sizeof(off)) != cudaSuccess
	    || cudaMalloc((void **)&g_legacy.flags_twin, 4) != cudaSuccess
	    || cudaMalloc((void **)&g_legacy.flags_plain, 4) != cudaSuccess
	    || cudaMalloc((void **)&g_legacy.amax, 4) != cudaSuccess
	    || cudaMemset(g_legacy.ctl, 0, sizeof(anni_control)) != cudaSuccess
	    || cudaMemcpy(g_legacy.seg_off, off, sizeof(off), cudaMemcpyHostToDevice) != cudaSuccess
	    || cudaMemcpy(g_legacy.flags_twin, &f_twin, 4, cudaMemcpyHostToDevice) != cudaSuccess
	    || cudaMemcpy(g_legacy.flags_plain, &f_plain, 4, cudaMemcpyHostToDevice) != cudaSuccess
	    || (g_legacy.blocks = anni_grid_blocks(ANNI_DT_F32, ANNI_DT_F32, 0)) < 1) {
		/* all or nothing: a half-built state must not pass for a ready one at the next call */
		(void)cudaGetLastError();
		cudaFree(g_legacy.ctl);
		cudaFree(g_legacy.seg_off);
		cudaFree(g_legacy.flags_twin);
		cudaFree(g_legacy.flags_plain);
		cudaFree(g_legacy.amax);
		memset(&g_legacy, 0, sizeof(g_legacy));
		return -1;
	}
	return 0;
}

void legacy_launch_base(anni_launch *la, uint64_t n)
{
	memset(la, 0, sizeof(*la));
	la->n = n;
	la->seg_off = g_legacy.seg_off;
	la->seg_flags = g_legacy.flags_plain;
	la->seg_amax = g_legacy.amax;
	la->seg_scale = g_legacy.amax;
	la->n_seg = 1;
	la->sc_log2 = 2;
	la->ctl = g_legacy.ctl;
}

}	/* namespace */

/* ---- device, memory, stream ------------------------------------------------ */

extern "C" int gpu_available(void)
{
	std::call_once(g_once, init_once);
	return g_have_gpu;
}

extern "C" const char *gpu_backend_name(void)
{
	return gpu_available() ? "anni_b200 (sm_100a)" : "cpu";
}

extern "C" int gpu_mem_info(size_t *free_bytes, size_t *total_bytes)
{
	size_t f = 0;
	size_t t = 0;
	int ok = gpu_available() && cudaMemGetInfo(&f, &t) == cudaSuccess;

	if (free_bytes)
		*free_bytes = ok ? f : 0;
	if (total_bytes)
		*total_bytes = ok ? t : 0;
	return ok ? 0 : -1;
}

extern "C" void gpu_set_sync_mode(int mode)
{
	g_sync_mode_v = mode;
}

extern "C" int gpu_sync_mode(void)
{
	return g_sync_mode_v;
}

extern "C" void gpu_set_compute_prec(int prec)
{
	g_prec = prec;
}

extern "C" void gpu_set_fp8(int on)
{
	g_fp8_on = on ? 1 : 0;
	g_fp8_dgrad_on = g_fp8_on;
}

extern "C" void gpu_set_fp8_dgrad(int on)
{
	g_fp8_dgrad_on = on ? 1 : 0;
}

extern "C" int gpu_fp8(void)
{
	return g_fp8_on;
}

extern "C" void gpu_device_sync(void)
{
	if (gpu_available())
		(void)cudaDeviceSynchronize();
}

/*
** Large blocks (the optimizer's flats, lang/lm_adam.c:217-311) come from compressible memory
** where the device has it: the gradient flat is left zeroed by every step, and zeroed lines
** then cost a fraction of their size on the way to HBM.  Data that does not compress costs the
** same as in plain memory.  Small blocks, and every block where compression is unavailable,
** are plain cudaMalloc memory.  g_arena_blocks remembers which is which for gpu_free.
*/
#define ANNI_COMPRESSIBLE_FROM	((size_t)8 << 20)

extern "C" void *gpu_malloc(size_t nbytes)
{
	void *p = NULL;
	size_t mapped = 0;
	std::lock_guard<std::mutex> hold(g_malloc_lock);

	if (!gpu_available() || nbytes == 0)
		return NULL;
	if (nbytes >= ANNI_COMPRESSIBLE_FROM && anni_arena_alloc(nbytes, &p, &mapped, NULL) == ANNI_OK) {
		g_arena_blocks[p] = mapped;
		return p;
	}
	(void)cudaGetLastError();
	p = NULL;
	if (cudaMalloc(&p, nbytes) != cudaSuccess) {
		(void)cudaGetLastError();
		return NULL;
	}
	return p;
}

extern "C" void gpu_free(void *p)
{
	std::lock_guard<std::mutex> hold(g_malloc_lock);

	if (!p || !gpu_available())
		return;
	auto it = g_arena_blocks.find(p);
	if (it != g_arena_blocks.end()) {
		(void)anni_arena_free(p, it->second);
		g_arena_blocks.erase(it);
		return;
	}
	(void)cudaFree(p);
}

extern "C" int gpu_memcpy_h2d(void *dst, const void *src, size_t nbytes)
{
	if (!dst || !src || !gpu_available())
		return -1;
	return cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyHostToDevice, g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_memcpy_d2h(void *dst, const void *src, size_t nbytes)
{
	if (!dst || !src || !gpu_available())
		return -1;
	if (cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, g_st) != cudaSuccess)
		return -1;
	return cudaStreamSynchronize(g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_host_pin(void *p, size_t nbytes)
{
	cudaError_t e;

	if (!p || !gpu_available())
		return -1;
	e = cudaHostRegister(p, nbytes, cudaHostRegisterDefault);
	if (e == cudaErrorHostMemoryAlreadyRegistered) {
		(void)cudaGetLastError();
		return 0;
	}
	if (e != cudaSuccess) {
		(void)cudaGetLastError();
		return 0;	/* pageable memory still copies correctly, only slower */
	}
	return 0;
}

extern "C" int gpu_memcpy_d2h_async(void *dst, const void *src, size_t nbytes)
{
	if (!dst || !src || !gpu_available())
		return -1;
	return cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_stream_sync(void)
{
	if (!gpu_available())
		return -1;
	return cudaStreamSynchronize(g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_memcpy_d2d(void *dst, const void *src, size_t nbytes)
{
	if (!dst || !src || !gpu_available())
		return -1;
	return cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToDevice, g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_memset(void *dst, int value, size_t nbytes)
{
	if (!dst || !gpu_available())
		return -1;
	return cudaMemsetAsync(dst, value, nbytes, g_st) == cudaSuccess ? 0 : -1;
}

extern "C" void gpu_host_forget(const void *host)
{
	if (host && gpu_available()) {
		/* a pinned registration must not outlive the allocation it covered */
		if (cudaHostUnregister((void *)host) != cudaSuccess)
			(void)cudaGetLastError();
	}
}

extern "C" const char *gpu_debug_last_error(void)
{
	cudaError_t e;

	if (!gpu_available())
		return "";
	e = cudaGetLastError();
	return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

extern "C" void gpu_op_prof_dump(void)
{
	static int on = -1;

	if (on < 0) {
		const char *e = getenv("ANN_OP_PROF");

		on = (e && e[0] == '1') ? 1 : 0;
	}
	if (on)
		fprintf(stderr, "[anni_b200] kernel launches so far: %llu\n",
		    (unsigned long long)anni_kernel_launches());
}

/* ---- the flat bf16 twin registry ---------------------------------------------- */

extern "C" void gpu_half_wt_invalidate(const ann_real_t *fp32_dev)
{
	(void)fp32_dev;
	g_wt_epoch++;	/* derived copies (packed QKV, fp8, host-vector caches) rebuild lazily */
}

extern "C" unsigned gpu_param_epoch(void)
{
	return g_wt_epoch;
}

extern "C" void gpu_adam_set_bf16_flat(void *bf16, const ann_real_t *fp32, int n)
{
	g_flat_bf16 = bf16;
	g_flat_fp32 = fp32;
	g_flat_n = bf16 && fp32 && n > 0 ? (size_t)n : 0;
}

extern "C" int gpu_adam_seed_bf16_flat(void *bf16, const ann_real_t *fp32, int n)
{
	if (!bf16 || !fp32 || n <= 0 || !gpu_available())
		return -1;
	return anni_launch_f32_to_bf16((uint16_t *)bf16, fp32, (uint64_t)n, g_st) == ANNI_OK ? 0 : -1;
}

extern "C" void *anni_half_wt_lookup(const ann_real_t *fp32_dev, size_t n)
{
	size_t off;

	if (!g_flat_n || !fp32_dev || fp32_dev < g_flat_fp32)
		return NULL;
	off = (size_t)(fp32_dev - g_flat_fp32);
	if (off >= g_flat_n || n > g_flat_n - off)
		return NULL;
	return (char *)g_flat_bf16 + off * 2;	/* same element offset, two bytes each */
}

/* ---- the optimizer's two device calls ------------------------------------------ */

extern "C" void gpu_adam_set_weight_decay(double wd)
{
	g_adam_wd = wd > 0.0 ? wd : 0.0;
}

extern "C" int anni_grad_sumsq64(const void *d_x, int dtype, unsigned long long n, double *out)
{
	anni_launch la;

	if (!d_x || n == 0 || !out || !gpu_available() || legacy_ready() != 0)
		return -1;
	if (dtype != ANNI_DT_F32 && dtype != ANNI_DT_BF16)
		return -1;
	legacy_launch_base(&la, n);
	la.grad = (void *)d_x;
	la.aligned = ((uintptr_t)d_x & 15) == 0;
	if (anni_launch_norm(&la, dtype, ANNI_DT_F32, g_legacy.blocks, g_st) != ANNI_OK)
		return -1;
	/* the reference returns the sum to the host with a blocking copy (gpu_cuda.cu:8532) */
	if (cudaMemcpyAsync(out, (char *)g_legacy.ctl + offsetof(anni_control, reduce), sizeof(double),
	    cudaMemcpyDeviceToHost, g_st) != cudaSuccess)
		return -1;
	return cudaStreamSynchronize(g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_grad_sumsq(const ann_real_t *d_x, int n, double *out)
{
	if (n <= 0)
		return -1;
	return anni_grad_sumsq64(d_x, ANNI_DT_F32, (unsigned long long)n, out);
}

extern "C" int anni_adam_step_dev64(ann_real_t *d_p, void *d_p_bf16, ann_real_t *d_g, ann_real_t *d_m,
	ann_real_t *d_v, unsigned long long n, double lr, double beta1, double beta2, double eps, int t,
	double grad_scale)
{
	anni_launch la;
	anni_optstep_hyper hp;
	const int twin = d_p_bf16 && g_prec == ANNI_GPU_PREC_BF16;

	if (!d_p || !d_g || !d_m || !d_v || n == 0 || !(lr > 0.0) || t < 1)
		return -1;
	if (!gpu_available() || legacy_ready() != 0)
		return -1;
	legacy_launch_base(&la, n);
	la.master = d_p;
	la.m = d_m;
	la.v = d_v;
	la.grad = d_g;
	la.twin16 = twin ? (uint16_t *)d_p_bf16 : NULL;
	la.seg_flags = twin ? g_legacy.flags_twin : g_legacy.flags_plain;
	la.aligned = (((uintptr_t)d_p | (uintptr_t)d_g | (uintptr_t)d_m | (uintptr_t)d_v
	    | (uintptr_t)la.twin16) & 15) == 0;
	memset(&hp, 0, sizeof(hp));
	hp.lr = lr;
	hp.beta1 = beta1;
	hp.beta2 = beta2;
	hp.eps = eps;
	hp.weight_decay = g_adam_wd;
	hp.grad_clip = 0.0;		/* the caller folded its clip factor into grad_scale */
	hp.grad_scale = grad_scale;
	hp.t = t;
	/* "d_grad is zeroed after" (gpu.h:125-127); with fp32 moments the double update term costs a few per cent */
	hp.flags = ANNI_STEP_ZERO_GRAD | ANNI_STEP_EXACT_UPDATE;
	if (anni_fill_hyper(&la, &hp) != ANNI_OK)
		return -1;		/* bias correction not positive, as gpu_cuda.cu:8681 */
	la.flags |= ANNI_LAUNCH_HOST_COEF;
	return anni_launch_update(&la, ANNI_DT_F32, ANNI_DT_F32, g_legacy.blocks, g_st) == ANNI_OK
	    ? 0 : -1;
}

extern "C" int gpu_adam_step_dev_bf16(ann_real_t *d_p, void *d_p_bf16, ann_real_t *d_g,
	ann_real_t *d_m, ann_real_t *d_v, int n, double lr, double beta1, double beta2, double eps,
	int t, double grad_scale)
{
	if (n <= 0)
		return -1;
	return anni_adam_step_dev64(d_p, d_p_bf16, d_g, d_m, d_v, (unsigned long long)n, lr, beta1,
	    beta2, eps, t, grad_scale);
}

/* y += a x on the device twins (gpu.h:299); host-authoritative operands are uploaded first. */
extern "C" int gpu_mat_axpy(anni_mat *y, double a, const anni_mat *x)
{
	size_t n;
	size_t nb;
	anni_mat *xm = (anni_mat *)x;
	anni_mat *ops[2];

	if (!y || !x || y->rows != x->rows || y->cols != x->cols || !gpu_available())
		return -1;
	n = (size_t)y->rows * (size_t)y->cols;
	nb = n * sizeof(float);
	if (n == 0)
		return -1;
	ops[0] = y;
	ops[1] = xm;
	for (int k = 0; k < 2; k++) {
		anni_mat *mt = ops[k];

		if (!mt->d_data) {
			mt->d_data = (float *)gpu_malloc(nb);
			if (!mt->d_data)
				return -1;
			mt->on_device = 0;
		}
		if (mt->on_device == 0) {	/* host is authoritative: bring it over */
			if (!mt->data || gpu_memcpy_h2d(mt->d_data, mt->data, nb) != 0)
				return -1;
			mt->on_device = 2;
		}
	}
	if (anni_launch_axpy(y->d_data, x->d_data, (float)a, n, g_st) != ANNI_OK)
		return -1;
	if (y->on_device != 3)
		y->on_device = 1;	/* device-authoritative; an aliased view stays aliased */
	if (g_sync_mode_v == ANNI_GPU_SYNC_EAGER)
		(void)cudaStreamSynchronize(g_st);
	return 0;
}

/* ---- everything else in num/gpu.h: not on the device ----------------------------- */

/*
** Forward/backward, inference and CUDA-graph entry points.  Only the symbol
** and the value it returns matter to the linker and to the callers (they fall
** back to their CPU code); argument lists are therefore left empty.  Values
** are those of the reference's stub backend.
*/
#define NOT_ON_DEVICE(name)	extern "C" int name() { return -1; }
#define ANSWERS_ZERO(name)	extern "C" int name() { return 0; }
#define NO_POINTER(name)	extern "C" void *name() { return NULL; }
#define NOTHING_TO_DO(name)	extern "C" void name() { }

NOT_ON_DEVICE(gpu_ce_fetch_mean)
NOT_ON_DEVICE(gpu_mat_mul)
NOT_ON_DEVICE(gpu_mat_mul_bias)
NOT_ON_DEVICE(gpu_mat_mul_res)
NOT_ON_DEVICE(gpu_mat_mul_bias_relu)
NOT_ON_DEVICE(gpu_mat_mul_bt)
NOT_ON_DEVICE(gpu_mat_mul_bt_acc)
NOT_ON_DEVICE(gpu_mat_mul_bt_twin)
NOT_ON_DEVICE(gpu_mat_mul_at)
NOT_ON_DEVICE(gpu_mat_outer_add)
NOT_ON_DEVICE(gpu_layernorm_backward)
NOT_ON_DEVICE(gpu_layernorm_backward_acc)
NOT_ON_DEVICE(gpu_layernorm_backward_x)
NOT_ON_DEVICE(gpu_layernorm_xhat)
NOT_ON_DEVICE(gpu_softmax_rows)
NOT_ON_DEVICE(gpu_softmax_bwd_rows)
NOT_ON_DEVICE(gpu_layernorm_forward_ex)
NOT_ON_DEVICE(gpu_bias_row_add)
NOT_ON_DEVICE(gpu_ce_delta_from_softmax)
NOT_ON_DEVICE(gpu_ce_softmax_delta_bf16)
ANSWERS_ZERO(gpu_ce_bias_fused)
NOT_ON_DEVICE(gpu_ce_bf16_delta_done)
NOT_ON_DEVICE(gpu_ce_nll_rows)
NOT_ON_DEVICE(gpu_posenc_add_packed)
NOT_ON_DEVICE(gpu_mat_col_sum_add)
NOT_ON_DEVICE(gpu_relu_backward)
NOT_ON_DEVICE(gpu_ffn_relu_bwd_fused)
ANSWERS_ZERO(gpu_act_bf16_only)
NOT_ON_DEVICE(gpu_attn_causal_fwd)
NOT_ON_DEVICE(gpu_attn_flash_fwd)
NOT_ON_DEVICE(gpu_attn_fa_fwd)
ANSWERS_ZERO(gpu_attn_fa_usable)
NOT_ON_DEVICE(gpu_attn_fa_bwd)
extern "C" int gpu_attn_qkv_bwd() { return 1; }	/* the stub's "not handled" answer for this call */
NOT_ON_DEVICE(gpu_attn_tiled_bwd)
NOT_ON_DEVICE(gpu_attn_causal_bwd)
NOT_ON_DEVICE(gpu_attn_tc_fwd)
NOT_ON_DEVICE(gpu_attn_tc_bwd)
NOT_ON_DEVICE(gpu_attn_qkv_fused)
NOT_ON_DEVICE(gpu_pack_seq_rows)
NOT_ON_DEVICE(gpu_unpack_seq_rows)
NOT_ON_DEVICE(gpu_ffn_w1_finish)
NOT_ON_DEVICE(gpu_mat_copy)
NOT_ON_DEVICE(gpu_mat_add)
NOT_ON_DEVICE(gpu_mat_add2)
NOT_ON_DEVICE(gpu_embed_lookup)
NOT_ON_DEVICE(gpu_embed_scatter)
NOT_ON_DEVICE(gpu_graph_begin)
NOT_ON_DEVICE(gpu_graph_end)
NOT_ON_DEVICE(gpu_graph_replay)
ANSWERS_ZERO(gpu_graph_replayable)
ANSWERS_ZERO(gpu_graph_supported)
NOT_ON_DEVICE(gpu_ids_stage)
NOT_ON_DEVICE(gpu_dec_set_layer)
NOT_ON_DEVICE(gpu_dec_set_io)
NOT_ON_DEVICE(gpu_dec_kv_load)
NOT_ON_DEVICE(gpu_dec_step)
NO_POINTER(gpu_host_alloc)
NO_POINTER(gpu_copy_stream)
NO_POINTER(gpu_ce_targets_staged)
NO_POINTER(gpu_dec_create)
NOTHING_TO_DO(gpu_grad_twins_clear)
NOTHING_TO_DO(gpu_attn_qkv_bf16_hint)
NOTHING_TO_DO(gpu_attn_set_seqlens)
NOTHING_TO_DO(gpu_host_free)
NOTHING_TO_DO(gpu_graph_destroy)
NOTHING_TO_DO(gpu_graph_set_mode)
NOTHING_TO_DO(gpu_ids_unstage)
NOTHING_TO_DO(gpu_dec_free)
