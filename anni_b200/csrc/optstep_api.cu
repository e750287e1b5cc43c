/*
** Host side of the packed-arena engine: life cycle, argument checks and the
** launch sequences behind the anni_optstep_* entry points of anni_b200.h.
** No arithmetic on parameters happens on the host; a missing device is an
** error, never a reason to compute on the CPU.
*/
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include "optstep_internal.h"

struct anni_optstep {
	anni_optstep_config	cfg;
	anni_launch		la;		/* buffers + tables, hyper filled per step */
	anni_control		*ctl;		/* device */
	int64_t			*d_seg_off;
	uint32_t		*d_seg_flags;
	float			*d_amax;
	float			*d_scale;
	uint32_t		*d_seg_done;	/* per-tensor arrival counters of the one-launch fp8 step */
	anni_seg_derived	*d_aux;		/* derived-twin table (anni_optstep_set_derived) */
	int64_t			*d_tile_prefix;	/* tiles before each tensor, transposed e4m3 twins */
	int64_t			n_tiles;
	int64_t			*h_seg_off;	/* host copies, for argument checks */
	uint32_t		*h_seg_flags;
	int			n_seg;
	int			has_fp8;
	int			bound;
	int			device;
	int			blocks_coop;
	int			blocks_split;
	int			blocks_rn;	/* grid of the fused reduce-scatter + norm kernel */
	int			fp8_pipe;	/* one-launch fp8 step: quantise behind the update (opt-in) */
	int			fp8_stream;
	/* ZeRO-1: this rank's full gradient arena, cleared by the update instead of the bound shard */
	void			*grad_arena;
	uint64_t		grad_arena_stride;
	int			grad_arena_parts;
};

static int derived_after_step(anni_optstep *h, const anni_launch *la, cudaStream_t st);

/* split form: the update clears the rank's full gradient arena, if one was named */
static void use_grad_arena(const anni_optstep *h, anni_launch *la)
{
	if (h->grad_arena && (la->flags & ANNI_STEP_ZERO_GRAD)) {
		la->zero_base = h->grad_arena;
		la->zero_stride = h->grad_arena_stride;
		la->zero_parts = h->grad_arena_parts;
	}
}

/*
** Which part of the named arena is this rank's own, i.e. which peer pointer lies inside it at a
** part boundary: the part's index, or -1.  *slot = that peer's position in the table.
*/
static int own_part(const anni_optstep *h, int *slot)
{
	const size_t gsz = h->cfg.grad_dtype == ANNI_DT_BF16 ? 2u : 4u;
	const uintptr_t base = (uintptr_t)h->grad_arena;
	const uintptr_t part = (uintptr_t)h->grad_arena_stride * gsz;

	if (!h->grad_arena || part == 0)
		return -1;
	for (int k = 0; k < h->la.n_peers; k++) {
		const uintptr_t p = (uintptr_t)h->la.peer_grad[k];

		if (p >= base && p < base + part * (uintptr_t)h->grad_arena_parts && (p - base) % part == 0) {
			if (slot)
				*slot = k;
			return (int)((p - base) / part);
		}
	}
	return -1;
}

/* ANNI_STEP_REDUCE_CLEARS_OWN on the reduce side: name the part to clear, or refuse */
static int reduce_clears_own(const anni_optstep *h, anni_launch *la)
{
	int slot = 0;

	la->own_clear = NULL;
	if (!(la->flags & ANNI_STEP_REDUCE_CLEARS_OWN))
		return ANNI_OK;
	if (!(la->flags & ANNI_STEP_ZERO_GRAD) || la->mc_grad || own_part(h, &slot) < 0)
		return ANNI_E_ARG;
	la->own_clear = const_cast<void *>(la->peer_grad[slot]);
	return ANNI_OK;
}

/* ... and on the update side: that part is done */
static int update_skips_own(const anni_optstep *h, anni_launch *la)
{
	int part;

	la->zero_done = 0;
	if (!(la->flags & ANNI_STEP_REDUCE_CLEARS_OWN))
		return ANNI_OK;
	part = own_part(h, NULL);
	if (!(la->flags & ANNI_STEP_ZERO_GRAD) || la->zero_parts < 1 || part < 0)
		return ANNI_E_ARG;
	la->zero_done = part + 1;
	return ANNI_OK;
}

/* ... and what lies beyond this shard's length in every part, which the update's walk never visits */
static int zero_arena_tail(const anni_optstep *h, const anni_launch *la, cudaStream_t st)
{
	if (la->zero_parts < 1 || h->cfg.shard_n >= h->grad_arena_stride)
		return ANNI_OK;
	return anni_launch_zero_tail(h->grad_arena, h->cfg.grad_dtype, h->cfg.shard_n, h->grad_arena_stride,
	    h->grad_arena_parts, st);
}

/* ANNI_B200_SUPERCHUNK=k: 2^k consecutive chunks per block per round (tuning knob). */
static int superchunk_log2(void)
{
	const char *e = getenv("ANNI_B200_SUPERCHUNK");
	int k = e ? atoi(e) : 2;

	return k < 0 ? 0 : (k > 20 ? 20 : k);
}

/*
** Launch geometry of the step kernels for the given dtypes on the current device: the
** persistent grid (the same for the one-launch and the split form, so that their block
** partials, and with them the norm's bits, agree) and the super-chunk size.  Every path that
** launches those kernels -- engines and the allocation-free entry point -- asks here, so they
** all honour the tuning knobs and report identical norms.
*/
extern "C" int anni_engine_geometry(int grad_dtype, int state_dtype, int *blocks, int *sc_log2)
{
	const char *e = getenv("ANNI_B200_BLOCKS_PER_SM");	/* fewer resident blocks than fit (tuning knob) */
	int coop = anni_grid_blocks(grad_dtype, state_dtype, 1);
	int split = anni_grid_blocks(grad_dtype, state_dtype, 0);
	int dev = 0;
	int sms = 0;

	if (coop < 1 || split < 1)
		return ANNI_E_CUDA;
	if (split < coop)
		coop = split;
	if (e && atoi(e) > 0 && cudaGetDevice(&dev) == cudaSuccess
	    && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess
	    && sms > 0 && atoi(e) * sms < coop)
		coop = atoi(e) * sms;
	if (blocks)
		*blocks = coop;
	if (sc_log2)
		*sc_log2 = superchunk_log2();
	return ANNI_OK;
}

static int check_cfg(const anni_optstep_config *c)
{
	int i;

	if (!c || c->shard_off > c->n_arena || c->shard_n > c->n_arena - c->shard_off)
		return ANNI_E_ARG;
	if ((c->grad_dtype != ANNI_DT_F32 && c->grad_dtype != ANNI_DT_BF16)
	    || (c->state_dtype != ANNI_DT_F32 && c->state_dtype != ANNI_DT_BF16))
		return ANNI_E_ARG;
	if (c->n_seg < 0 || (c->n_seg > 0 && (!c->seg_off || !c->seg_flags)))
		return ANNI_E_ARG;
	if (c->n_seg > 0) {
		if (c->seg_off[0] != 0 || (uint64_t)c->seg_off[c->n_seg] != c->n_arena)
			return ANNI_E_ARG;
		for (i = 0; i < c->n_seg; i++)
			if (c->seg_off[i + 1] < c->seg_off[i])
				return ANNI_E_ARG;
	}
	return ANNI_OK;
}

extern "C" int anni_optstep_create(const anni_optstep_config *cfg, anni_optstep **out)
{
	anni_optstep *h;
	int64_t one_off[2];
	uint32_t one_flag = ANNI_SEG_WD | ANNI_SEG_TWIN_BF16;
	const int64_t *off;
	const uint32_t *flg;
	int rc;
	int i;

	if (!out)
		return ANNI_E_ARG;
	*out = NULL;
	rc = check_cfg(cfg);
	if (rc != ANNI_OK)
		return rc;
	h = (anni_optstep *)calloc(1, sizeof(*h));
	if (!h)
		return ANNI_E_NOMEM;
	h->cfg = *cfg;
	h->cfg.seg_off = NULL;
	h->cfg.seg_flags = NULL;
	if (cudaGetDevice(&h->device) != cudaSuccess) {
		free(h);
		return ANNI_E_CUDA;
	}
	if (cfg->n_seg > 0) {
		h->n_seg = cfg->n_seg;
		off = cfg->seg_off;
		flg = cfg->seg_flags;
	} else {
		h->n_seg = 1;
		one_off[0] = 0;
		one_off[1] = (int64_t)cfg->n_arena;
		off = one_off;
		flg = &one_flag;
	}
	for (i = 0; i < h->n_seg; i++)
		if (flg[i] & ANNI_SEG_TWIN_FP8)
			h->has_fp8 = 1;
	h->h_seg_off = (int64_t *)malloc((size_t)(h->n_seg + 1) * sizeof(int64_t));
	h->h_seg_flags = (uint32_t *)malloc((size_t)h->n_seg * sizeof(uint32_t));
	if (!h->h_seg_off || !h->h_seg_flags) {
		anni_optstep_destroy(h);
		return ANNI_E_NOMEM;
	}
	memcpy(h->h_seg_off, off, (size_t)(h->n_seg + 1) * sizeof(int64_t));
	memcpy(h->h_seg_flags, flg, (size_t)h->n_seg * sizeof(uint32_t));
	if (cudaMalloc((void **)&h->ctl, sizeof(anni_control)) != cudaSuccess
	    || cudaMalloc((void **)&h->d_seg_off, (size_t)(h->n_seg + 1) * sizeof(int64_t)) != cudaSuccess
	    || cudaMalloc((void **)&h->d_seg_flags, (size_t)h->n_seg * sizeof(uint32_t)) != cudaSuccess
	    || cudaMalloc((void **)&h->d_amax, (size_t)h->n_seg * sizeof(float)) != cudaSuccess
	    || cudaMalloc((void **)&h->d_scale, (size_t)h->n_seg * sizeof(float)) != cudaSuccess
	    || cudaMalloc((void **)&h->d_seg_done, (size_t)h->n_seg * sizeof(uint32_t)) != cudaSuccess
	    || cudaMemset(h->d_seg_done, 0, (size_t)h->n_seg * sizeof(uint32_t)) != cudaSuccess
	    || cudaMemset(h->ctl, 0, sizeof(anni_control)) != cudaSuccess
	    || cudaMemset(h->d_amax, 0, (size_t)h->n_seg * sizeof(float)) != cudaSuccess
	    || cudaMemset(h->d_scale, 0, (size_t)h->n_seg * sizeof(float)) != cudaSuccess
	    || cudaMemcpy(h->d_seg_off, off, (size_t)(h->n_seg + 1) * sizeof(int64_t),
	    cudaMemcpyHostToDevice) != cudaSuccess
	    || cudaMemcpy(h->d_seg_flags, flg, (size_t)h->n_seg * sizeof(uint32_t),
	    cudaMemcpyHostToDevice) != cudaSuccess) {
		anni_optstep_destroy(h);
		return ANNI_E_CUDA;
	}
	if (anni_engine_geometry(cfg->grad_dtype, cfg->state_dtype, &h->blocks_coop, &h->la.sc_log2) != ANNI_OK) {
		anni_optstep_destroy(h);
		return ANNI_E_CUDA;
	}
	h->blocks_split = h->blocks_coop;
	h->blocks_rn = h->blocks_split;
	{
		/* ANNI_B200_RN_BLOCKS_PER_SM=k: resident blocks of the reduce-scatter + norm kernel (tuning knob) */
		const char *e = getenv("ANNI_B200_RN_BLOCKS_PER_SM");
		int sms = 0;

		if (e && atoi(e) > 0 && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount,
		    h->device) == cudaSuccess && sms > 0 && atoi(e) * sms < h->blocks_rn)
			h->blocks_rn = atoi(e) * sms;
	}
	h->la.n = cfg->shard_n;
	h->la.arena_off = cfg->shard_off;
	h->la.seg_off = h->d_seg_off;
	h->la.seg_flags = h->d_seg_flags;
	h->la.seg_amax = h->d_amax;
	h->la.seg_scale = h->d_scale;
	h->la.seg_done = h->d_seg_done;
	h->la.n_seg = h->n_seg;
	h->la.ctl = h->ctl;
	{
		/*
		** ANNI_B200_FP8_PIPE=1: quantise tensor by tensor behind the update instead of in a phase of
		** its own after a second grid barrier.  Off by default: it takes the quantiser's reads off
		** HBM (91 % of them hit the L2) but not off the path between the SMs and the L2, and its
		** bookkeeping costs more than the DRAM time it saves (555 M parameters: 2.58 against 2.42 ms).
		*/
		const char *e = getenv("ANNI_B200_FP8_PIPE");

		h->fp8_pipe = e && e[0] == '1';
		/* ANNI_B200_FP8_LAG=k: quantising trips per round while several tensors are waiting (tuning knob) */
		e = getenv("ANNI_B200_FP8_LAG");
		h->la.pipe_lag = e && atoi(e) > 0 ? atoi(e) : ANNI_PIPE_LAG;
		e = getenv("ANNI_B200_FP8_STREAM");
		h->fp8_stream = e && e[0] == '1';
	}
	*out = h;
	return ANNI_OK;
}

extern "C" void anni_optstep_destroy(anni_optstep *h)
{
	if (!h)
		return;
	cudaFree(h->ctl);
	cudaFree(h->d_seg_off);
	cudaFree(h->d_seg_flags);
	cudaFree(h->d_amax);
	cudaFree(h->d_scale);
	cudaFree(h->d_seg_done);
	cudaFree(h->d_aux);
	cudaFree(h->d_tile_prefix);
	free(h->h_seg_off);
	free(h->h_seg_flags);
	free(h);
}

extern "C" int anni_optstep_bind(anni_optstep *h, const anni_optstep_buffers *b)
{
	uintptr_t bits;

	if (!h || !b)
		return ANNI_E_ARG;
	if (h->cfg.shard_n > 0 && (!b->master || !b->m || !b->v || !b->grad))
		return ANNI_E_ARG;
	if (h->has_fp8 && h->cfg.shard_n > 0 && !b->twin_fp8)
		return ANNI_E_ARG;
	bits = (uintptr_t)b->master | (uintptr_t)b->m | (uintptr_t)b->v | (uintptr_t)b->grad
	    | (uintptr_t)b->twin_bf16 | (uintptr_t)b->twin_fp8;
	h->la.master = b->master;
	h->la.m = b->m;
	h->la.v = b->v;
	h->la.grad = b->grad;
	h->la.twin16 = (uint16_t *)b->twin_bf16;
	h->la.twin8 = (uint8_t *)b->twin_fp8;
	h->la.aligned = (bits & 15) == 0;
	h->bound = 1;
	return ANNI_OK;
}

static int prepare(anni_optstep *h, const anni_optstep_hyper *hp, anni_launch *la)
{
	int rc;

	if (!h || !hp || !h->bound)
		return ANNI_E_ARG;
	*la = h->la;
	la->flags = h->has_fp8 ? ANNI_LAUNCH_HAS_FP8 : 0;
	rc = anni_fill_hyper(la, hp);
	return rc;
}

extern "C" int anni_optstep_step(anni_optstep *h, const anni_optstep_hyper *hp, void *stream)
{
	anni_launch la;
	cudaStream_t st = (cudaStream_t)stream;
	int rc = prepare(h, hp, &la);

	if (rc != ANNI_OK)
		return rc;
	if (h->has_fp8 && h->fp8_pipe)
		la.flags |= ANNI_LAUNCH_FP8_PIPE | (h->fp8_stream ? ANNI_LAUNCH_PIPE_STREAM : 0);	/* the kernel clears amax and counters itself: ONE launch */
	else if (h->has_fp8 && cudaMemsetAsync(h->d_amax, 0, (size_t)h->n_seg * sizeof(float), st)
	    != cudaSuccess)
		return ANNI_E_CUDA;
	{
		const int slot = anni_op_begin(ANNI_OP_ADAM, st);

		rc = anni_launch_fused(&la, h->cfg.grad_dtype, h->cfg.state_dtype, h->blocks_coop, st);
		if (rc == ANNI_OK)
			rc = derived_after_step(h, &la, st);
		anni_op_end(slot, st);
	}
	return rc;
}

extern "C" int anni_optstep_norm(anni_optstep *h, const anni_optstep_hyper *hp, void *stream)
{
	anni_launch la;
	int rc = prepare(h, hp, &la);

	if (rc != ANNI_OK)
		return rc;
	{
		const int slot = anni_op_begin(ANNI_OP_SUMSQ, stream);

		rc = anni_launch_norm(&la, h->cfg.grad_dtype, h->cfg.state_dtype, h->blocks_split, (cudaStream_t)stream);
		anni_op_end(slot, stream);
	}
	return rc;
}

extern "C" int anni_optstep_update(anni_optstep *h, const anni_optstep_hyper *hp, void *stream)
{
	anni_launch la;
	cudaStream_t st = (cudaStream_t)stream;
	int rc = prepare(h, hp, &la);

	if (rc != ANNI_OK)
		return rc;
	if (h->has_fp8 && cudaMemsetAsync(h->d_amax, 0, (size_t)h->n_seg * sizeof(float), st)
	    != cudaSuccess)
		return ANNI_E_CUDA;
	use_grad_arena(h, &la);
	rc = update_skips_own(h, &la);
	if (rc != ANNI_OK)
		return rc;
	{
		const int slot = anni_op_begin(ANNI_OP_ADAM, st);

		rc = anni_launch_update(&la, h->cfg.grad_dtype, h->cfg.state_dtype, h->blocks_split, st);
		if (rc == ANNI_OK)
			rc = zero_arena_tail(h, &la, st);
		anni_op_end(slot, st);
	}
	return rc;
}

extern "C" int anni_optstep_step_with_sumsq(anni_optstep *h, const anni_optstep_hyper *hp,
	const double *d_sumsq, void *stream)
{
	cudaStream_t st = (cudaStream_t)stream;
	int rc;

	if (!h || !hp || !d_sumsq || !h->bound)
		return ANNI_E_ARG;
	if (cudaMemcpyAsync(anni_optstep_reduce_buffer(h), d_sumsq, 2 * sizeof(double), cudaMemcpyDeviceToDevice,
	    st) != cudaSuccess)
		return ANNI_E_CUDA;
	rc = anni_optstep_update(h, hp, stream);
	if (rc == ANNI_OK && h->has_fp8)
		rc = anni_optstep_quantize(h, stream);
	return rc;
}

extern "C" int anni_optstep_set_derived(anni_optstep *h, const anni_seg_derived *aux, void *qkv_packed,
	void *fp8_t)
{
	int64_t *prefix;
	int64_t tiles = 0;
	int any_pack = 0;
	int any_t = 0;
	int i;

	if (!h)
		return ANNI_E_ARG;
	cudaFree(h->d_aux);
	cudaFree(h->d_tile_prefix);
	h->d_aux = NULL;
	h->d_tile_prefix = NULL;
	h->n_tiles = 0;
	h->la.seg_aux = NULL;
	h->la.qkv_packed = NULL;
	h->la.fp8_t = NULL;
	if (!aux)
		return ANNI_OK;
	if (h->cfg.shard_off != 0 || h->cfg.shard_n != h->cfg.n_arena)
		return ANNI_E_ARG;	/* whole-arena engines only */
	prefix = (int64_t *)malloc((size_t)(h->n_seg + 1) * sizeof(int64_t));
	if (!prefix)
		return ANNI_E_NOMEM;
	for (i = 0; i < h->n_seg; i++) {
		const int64_t n = h->h_seg_off[i + 1] - h->h_seg_off[i];
		const int shaped = aux[i].rows > 0 && aux[i].cols > 0;

		prefix[i] = tiles;
		if (shaped && (int64_t)aux[i].rows * aux[i].cols != n)
			goto bad;
		if (aux[i].pack_ld != 0) {
			/* vector stores of four elements must stay inside one row, 8-byte aligned */
			if (!shaped || !(h->h_seg_flags[i] & ANNI_SEG_TWIN_BF16) || aux[i].cols % 4 != 0
			    || aux[i].pack_ld % 4 != 0 || aux[i].pack_off % 4 != 0 || aux[i].pack_off < 0
			    || aux[i].pack_ld < aux[i].cols)
				goto bad;
			any_pack = 1;
		}
		if (aux[i].fp8_t_off >= 0) {
			if (!shaped || !(h->h_seg_flags[i] & ANNI_SEG_TWIN_FP8))
				goto bad;
			tiles += (int64_t)((aux[i].rows + ANNI_TT_R - 1) / ANNI_TT_R)
			    * ((aux[i].cols + ANNI_TT_C - 1) / ANNI_TT_C);
			any_t = 1;
		}
	}
	prefix[h->n_seg] = tiles;
	if ((any_pack && !qkv_packed) || (any_t && !fp8_t))
		goto bad;
	if (cudaMalloc((void **)&h->d_aux, (size_t)h->n_seg * sizeof(anni_seg_derived)) != cudaSuccess
	    || cudaMalloc((void **)&h->d_tile_prefix, (size_t)(h->n_seg + 1) * sizeof(int64_t)) != cudaSuccess
	    || cudaMemcpy(h->d_aux, aux, (size_t)h->n_seg * sizeof(anni_seg_derived),
	    cudaMemcpyHostToDevice) != cudaSuccess
	    || cudaMemcpy(h->d_tile_prefix, prefix, (size_t)(h->n_seg + 1) * sizeof(int64_t),
	    cudaMemcpyHostToDevice) != cudaSuccess) {
		free(prefix);
		return ANNI_E_CUDA;
	}
	free(prefix);
	h->n_tiles = tiles;
	h->la.seg_aux = h->d_aux;
	h->la.qkv_packed = (uint16_t *)qkv_packed;
	h->la.fp8_t = (uint8_t *)fp8_t;
	return ANNI_OK;
bad:
	free(prefix);
	return ANNI_E_ARG;
}

/* the transposed e4m3 twins: one more launch after the step's own quantise phase */
static int derived_after_step(anni_optstep *h, const anni_launch *la, cudaStream_t st)
{
	if (h->n_tiles <= 0)
		return ANNI_OK;
	return anni_launch_quantize_transposed(la, h->d_tile_prefix, h->n_tiles, h->blocks_split, st);
}

extern "C" int anni_optstep_set_peers(anni_optstep *h, const void *const *peer_grad,
	void *const *peer_twin, void *const *peer_twin_fp8, int n_peers, uint64_t arena_off_padded)
{
	const size_t gsz = h && h->cfg.grad_dtype == ANNI_DT_BF16 ? 2u : 4u;
	uintptr_t bits = 0;
	int k;

	if (!h || n_peers < 0 || n_peers > ANNI_MAX_PEERS)
		return ANNI_E_ARG;
	h->la.mc_grad = NULL;
	h->la.mc_twin = NULL;
	h->la.mc_twin8 = NULL;
	if (n_peers == 0) {
		h->la.n_peers = 0;
		return ANNI_OK;
	}
	if (!peer_grad || !peer_twin || (h->has_fp8 && !peer_twin_fp8))
		return ANNI_E_ARG;
	for (k = 0; k < n_peers; k++) {
		if (!peer_grad[k] || !peer_twin[k] || (h->has_fp8 && !peer_twin_fp8[k]))
			return ANNI_E_ARG;
		h->la.peer_grad[k] = (const char *)peer_grad[k] + arena_off_padded * gsz;
		h->la.twin_peer[k] = (uint16_t *)peer_twin[k] + arena_off_padded;
		h->la.twin8_peer[k] = h->has_fp8 ? (uint8_t *)peer_twin_fp8[k] + arena_off_padded : NULL;
		bits |= (uintptr_t)h->la.peer_grad[k] | (uintptr_t)h->la.twin_peer[k]
		    | (uintptr_t)h->la.twin8_peer[k];
	}
	if (bits & 15)
		return ANNI_E_ARG;	/* peer arenas and the shard offset must keep 16-byte alignment */
	h->la.n_peers = n_peers;
	return ANNI_OK;
}

extern "C" int anni_optstep_set_multicast(anni_optstep *h, const void *mc_grad, void *mc_twin,
	void *mc_twin_fp8, uint64_t arena_off_padded)
{
	const size_t gsz = h && h->cfg.grad_dtype == ANNI_DT_BF16 ? 2u : 4u;

	if (!h || h->la.n_peers < 1)
		return ANNI_E_ARG;	/* peers first: the element-wise paths still use them */
	h->la.mc_grad = mc_grad ? (const char *)mc_grad + arena_off_padded * gsz : NULL;
	h->la.mc_twin = mc_twin ? (uint16_t *)mc_twin + arena_off_padded : NULL;
	h->la.mc_twin8 = (mc_twin_fp8 && h->has_fp8) ? (uint8_t *)mc_twin_fp8 + arena_off_padded : NULL;
	if (((uintptr_t)h->la.mc_grad | (uintptr_t)h->la.mc_twin | (uintptr_t)h->la.mc_twin8) & 15)
		return ANNI_E_ARG;
	return ANNI_OK;
}

extern "C" int anni_optstep_rotate_peers(anni_optstep *h, int first)
{
	const void *g[ANNI_MAX_PEERS];
	uint16_t *t[ANNI_MAX_PEERS];
	uint8_t *t8[ANNI_MAX_PEERS];
	const int np = h ? h->la.n_peers : 0;
	int k;

	if (!h || np < 1 || first < 0 || first >= np)
		return ANNI_E_ARG;
	for (k = 0; k < np; k++) {
		g[k] = h->la.peer_grad[(first + k) % np];
		t[k] = h->la.twin_peer[(first + k) % np];
		t8[k] = h->la.twin8_peer[(first + k) % np];
	}
	for (k = 0; k < np; k++) {
		h->la.peer_grad[k] = g[k];
		h->la.twin_peer[k] = t[k];
		h->la.twin8_peer[k] = t8[k];
	}
	return ANNI_OK;
}

extern "C" int anni_optstep_set_grad_arena(anni_optstep *h, void *arena, uint64_t stride, int parts)
{
	if (!h)
		return ANNI_E_ARG;
	if (!arena) {
		h->grad_arena = NULL;
		h->grad_arena_stride = 0;
		h->grad_arena_parts = 0;
		return ANNI_OK;
	}
	/* every part must hold this shard, and vector stores need part bases that keep 16-byte alignment */
	if (parts < 1 || parts > ANNI_MAX_PEERS || stride < h->cfg.shard_n || (stride & 7u) != 0
	    || ((uintptr_t)arena & 15) != 0)
		return ANNI_E_ARG;
	h->grad_arena = arena;
	h->grad_arena_stride = stride;
	h->grad_arena_parts = parts;
	return ANNI_OK;
}

extern "C" int anni_optstep_reduce_norm(anni_optstep *h, const anni_optstep_hyper *hp, void *stream)
{
	anni_launch la;
	int rc = prepare(h, hp, &la);

	if (rc != ANNI_OK)
		return rc;
	if (la.n_peers < 1)
		return ANNI_E_ARG;
	rc = reduce_clears_own(h, &la);
	if (rc != ANNI_OK)
		return rc;
	return anni_launch_reduce_norm(&la, h->cfg.grad_dtype, h->blocks_rn, (cudaStream_t)stream);
}

/* a launch description restricted to elements [off, off + n) of the shard */
static int restrict_range(const anni_optstep *h, anni_launch *la, uint64_t off, uint64_t n)
{
	const size_t gsz = h->cfg.grad_dtype == ANNI_DT_BF16 ? 2u : 4u;
	const size_t ssz = h->cfg.state_dtype == ANNI_DT_BF16 ? 2u : 4u;
	int k;

	if ((off & 4095u) != 0 || off > h->cfg.shard_n || n > h->cfg.shard_n - off)
		return ANNI_E_ARG;
	la->n = n;
	la->arena_off += off;
	la->master += off;
	la->m = (char *)la->m + off * ssz;
	la->v = (char *)la->v + off * ssz;
	la->grad = (char *)la->grad + off * gsz;
	if (la->twin16)
		la->twin16 += off;
	if (la->twin8)
		la->twin8 += off;
	for (k = 0; k < la->n_peers; k++) {
		la->peer_grad[k] = (const char *)la->peer_grad[k] + off * gsz;
		la->twin_peer[k] += off;
		if (la->twin8_peer[k])
			la->twin8_peer[k] += off;
	}
	if (la->zero_base)
		la->zero_base = (char *)la->zero_base + off * gsz;
	if (la->own_clear)
		la->own_clear = (char *)la->own_clear + off * gsz;
	if (la->mc_grad)
		la->mc_grad = (const char *)la->mc_grad + off * gsz;
	if (la->mc_twin)
		la->mc_twin += off;
	if (la->mc_twin8)
		la->mc_twin8 += off;
	return ANNI_OK;
}

extern "C" int anni_optstep_reduce_norm_range(anni_optstep *h, const anni_optstep_hyper *hp,
	uint64_t elem_off, uint64_t elem_n, int flags, void *stream)
{
	anni_launch la;
	int rc = prepare(h, hp, &la);

	if (rc != ANNI_OK)
		return rc;
	if (la.n_peers < 1)
		return ANNI_E_ARG;
	rc = reduce_clears_own(h, &la);
	if (rc != ANNI_OK)
		return rc;
	rc = restrict_range(h, &la, elem_off, elem_n);
	if (rc != ANNI_OK)
		return rc;
	if (flags & ANNI_RANGE_ACCUMULATE)
		la.flags |= ANNI_LAUNCH_ACCUMULATE;
	return anni_launch_reduce_norm(&la, h->cfg.grad_dtype, h->blocks_rn, (cudaStream_t)stream);
}

extern "C" int anni_optstep_update_range(anni_optstep *h, const anni_optstep_hyper *hp,
	uint64_t elem_off, uint64_t elem_n, int flags, void *stream)
{
	anni_launch la;
	cudaStream_t st = (cudaStream_t)stream;
	int rc = prepare(h, hp, &la);

	if (rc != ANNI_OK)
		return rc;
	if (la.seg_aux)
		return ANNI_E_ARG;	/* derived twins are a whole-arena, one-GPU feature */
	use_grad_arena(h, &la);
	rc = update_skips_own(h, &la);
	if (rc != ANNI_OK)
		return rc;
	rc = restrict_range(h, &la, elem_off, elem_n);
	if (rc != ANNI_OK)
		return rc;
	if (flags & ANNI_RANGE_LOCAL_TWINS) {
		la.n_peers = 0;
		la.mc_twin = NULL;
		la.mc_twin8 = NULL;
	}
	if (!(flags & ANNI_RANGE_LAST))
		la.flags |= ANNI_LAUNCH_NO_EPILOGUE;
	if ((flags & ANNI_RANGE_FIRST) && h->has_fp8
	    && cudaMemsetAsync(h->d_amax, 0, (size_t)h->n_seg * sizeof(float), st) != cudaSuccess)
		return ANNI_E_CUDA;
	rc = anni_launch_update(&la, h->cfg.grad_dtype, h->cfg.state_dtype, h->blocks_split, st);
	if (rc != ANNI_OK || !(flags & ANNI_RANGE_LAST))
		return rc;
	return zero_arena_tail(h, &la, st);
}

extern "C" int anni_peer_copy(void *dst, const void *src, size_t nbytes, void *stream)
{
	if (!dst || !src)
		return ANNI_E_ARG;
	if (nbytes == 0)
		return ANNI_OK;
	return cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDefault, (cudaStream_t)stream) == cudaSuccess
	    ? ANNI_OK : ANNI_E_CUDA;
}

extern "C" int anni_optstep_quantize(anni_optstep *h, void *stream)
{
	return anni_optstep_quantize_ex(h, 0, stream);
}

extern "C" int anni_optstep_quantize_ex(anni_optstep *h, int flags, void *stream)
{
	anni_launch la;
	int rc;

	if (!h || !h->bound)
		return ANNI_E_ARG;
	if (!h->has_fp8)
		return ANNI_OK;
	la = h->la;
	la.flags = ANNI_LAUNCH_HAS_FP8;
	if (flags & ANNI_RANGE_LOCAL_TWINS) {
		la.n_peers = 0;
		la.mc_twin8 = NULL;
	}
	rc = anni_launch_quantize(&la, h->blocks_split, (cudaStream_t)stream);
	return rc != ANNI_OK ? rc : derived_after_step(h, &la, (cudaStream_t)stream);
}

extern "C" int anni_optstep_selftest_barrier_timeout(anni_optstep *h, unsigned max_polls, void *stream)
{
	if (!h)
		return ANNI_E_ARG;
	return anni_launch_barrier_timeout(h->ctl, h->blocks_coop, max_polls, (cudaStream_t)stream);
}

extern "C" double *anni_optstep_reduce_buffer(anni_optstep *h)
{
	return h ? (double *)((char *)h->ctl + offsetof(anni_control, reduce)) : NULL;
}

extern "C" float *anni_optstep_amax_buffer(anni_optstep *h)
{
	return h ? h->d_amax : NULL;
}

extern "C" float *anni_optstep_scale_buffer(anni_optstep *h)
{
	return h ? h->d_scale : NULL;
}

extern "C" int anni_optstep_status_read(anni_optstep *h, anni_optstep_status *out, void *stream)
{
	anni_control head;	/* only the scalars in front of partials[] are copied */
	const size_t nb = offsetof(anni_control, partials);

	if (!h || !out)
		return ANNI_E_ARG;
	if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess
	    || cudaMemcpy(&head, h->ctl, nb, cudaMemcpyDeviceToHost) != cudaSuccess)
		return ANNI_E_CUDA;
	out->sumsq = head.reduce[0];
	out->norm = head.norm;
	out->eff_scale = head.eff_scale;
	out->loss_scale = head.loss_scale;
	out->skipped = head.skipped;
	out->error = head.error;
	out->good_steps = head.good_steps;
	out->steps_done = head.steps_done;
	if (head.error != 0) {
		/* a bounded wait gave up: clear the counters so the engine can be used again */
		head.error = 0;
		head.bar_count = 0;
		head.norm_ticket = 0;
		head.done_ticket = 0;
		if (cudaMemcpy(h->ctl, &head, nb, cudaMemcpyHostToDevice) != cudaSuccess)
			return ANNI_E_CUDA;
	}
	return ANNI_OK;
}

extern "C" int anni_optstep_loss_scale_init(anni_optstep *h, double scale, int growth_interval,
	double growth, double backoff, double min_scale, double max_scale)
{
	anni_control head;
	const size_t nb = offsetof(anni_control, partials);

	if (!h)
		return ANNI_E_ARG;
	if (cudaDeviceSynchronize() != cudaSuccess
	    || cudaMemcpy(&head, h->ctl, nb, cudaMemcpyDeviceToHost) != cudaSuccess)
		return ANNI_E_CUDA;
	head.loss_scale = scale > 0.0 ? scale : 0.0;
	head.ls_interval = growth_interval;
	head.ls_growth = growth;
	head.ls_backoff = backoff;
	head.ls_min = min_scale;
	head.ls_max = max_scale;
	head.good_steps = 0;
	return cudaMemcpy(h->ctl, &head, nb, cudaMemcpyHostToDevice) == cudaSuccess
	    ? ANNI_OK : ANNI_E_CUDA;
}

/* Polls the blocks of the one-launch fp8 step have spent waiting for each other since the last call (diagnostics). */
extern "C" long long anni_optstep_pipe_polls(anni_optstep *h, void *stream)
{
	uint32_t v = 0;
	const uint32_t zero = 0;
	char *p = h ? (char *)h->ctl + offsetof(anni_control, pipe_polls) : NULL;

	if (!h || cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess
	    || cudaMemcpy(&v, p, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess
	    || cudaMemcpy(p, &zero, sizeof(zero), cudaMemcpyHostToDevice) != cudaSuccess)
		return -1;
	return (long long)v;
}

extern "C" int anni_optstep_grid(anni_optstep *h, int *blocks, int *threads)
{
	if (!h)
		return ANNI_E_ARG;
	if (blocks)
		*blocks = h->blocks_coop;
	if (threads)
		*threads = ANNI_THREADS;
	return ANNI_OK;
}
