/*
** ZeRO-1 step for a C trainer (anni_zero1.h): the host-side sequence around the shard engine.
** The two big collectives live inside the kernels (peer mode) or are NCCL's (NCCL mode); what
** goes through NCCL either way are the two-double all-reduce of the norm, the per-tensor amax
** and two one-float exchanges that order the ranks.  NCCL is bound at run time, so that the
** library loads where it is absent; nothing here touches parameters on the host.
*/
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <mutex>
#include "anni_zero1.h"
#include "optstep_internal.h"

namespace {

/* the slice of NCCL's C interface used here (nccl.h: enum values are part of its ABI) */
struct nccl_uid {
	char	internal[ANNI_ZERO1_UNIQUE_ID_BYTES];
};
enum { NCCL_UINT8 = 1, NCCL_FLOAT32 = 7, NCCL_FLOAT64 = 8, NCCL_BFLOAT16 = 9 };
enum { NCCL_SUM = 0, NCCL_MAX = 2 };

typedef int (*fn_get_unique_id)(nccl_uid *);
typedef int (*fn_comm_init_rank)(void **, int, nccl_uid, int);
typedef int (*fn_comm_destroy)(void *);
typedef int (*fn_all_reduce)(const void *, void *, size_t, int, int, void *, cudaStream_t);
typedef int (*fn_reduce_scatter)(const void *, void *, size_t, int, int, void *, cudaStream_t);
typedef int (*fn_all_gather)(const void *, void *, size_t, int, void *, cudaStream_t);

struct nccl_api {
	fn_get_unique_id	get_unique_id;
	fn_comm_init_rank	comm_init_rank;
	fn_comm_destroy		comm_destroy;
	fn_all_reduce		all_reduce;
	fn_reduce_scatter	reduce_scatter;
	fn_all_gather		all_gather;
	int			ok;
} g_nccl;
std::once_flag g_nccl_once;

void nccl_resolve(void)
{
	/* the copy already in the process first (a communicator handed in was made by it) */
	void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);

	if (!h)
		h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
	if (!h)
		h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
	if (!h)
		return;
	g_nccl.get_unique_id = (fn_get_unique_id)dlsym(h, "ncclGetUniqueId");
	g_nccl.comm_init_rank = (fn_comm_init_rank)dlsym(h, "ncclCommInitRank");
	g_nccl.comm_destroy = (fn_comm_destroy)dlsym(h, "ncclCommDestroy");
	g_nccl.all_reduce = (fn_all_reduce)dlsym(h, "ncclAllReduce");
	g_nccl.reduce_scatter = (fn_reduce_scatter)dlsym(h, "ncclReduceScatter");
	g_nccl.all_gather = (fn_all_gather)dlsym(h, "ncclAllGather");
	g_nccl.ok = g_nccl.get_unique_id && g_nccl.comm_init_rank && g_nccl.comm_destroy
	    && g_nccl.all_reduce && g_nccl.reduce_scatter && g_nccl.all_gather;
}

const nccl_api *nccl(void)
{
	std::call_once(g_nccl_once, nccl_resolve);
	return g_nccl.ok ? &g_nccl : NULL;
}

}	/* namespace */

struct anni_zero1 {
	anni_optstep	*eng;
	void		*comm;
	int		rank;
	int		world;
	int		grad_dtype;
	int		n_seg;		/* entries of the amax buffer */
	int		has_fp8;
	int		peer;		/* peer mode */
	uint64_t	per;		/* elements per shard, padding included */
	uint64_t	shard_off;
	uint64_t	shard_n;
	void		*grad_arena;
	void		*twin_arena;
	void		*twin_fp8_arena;
	void		*grad_shard;
	anni_optstep_buffers	bufs;	/* as bound */
	void		*peer_twin[ANNI_MAX_PEERS];
	void		*peer_twin8[ANNI_MAX_PEERS];
	const void	*mc_grad;
	void		*mc_twin;
	void		*mc_twin8;
	int		mc_on;		/* the reduce and the twin stores go through the multicast addresses */
	int		clear_own;	/* the reduce clears this rank's own part of the arena (knob) */
	float		*d_tick;	/* one float: the ordering exchanges */
	int		bound;
};

extern "C" int anni_zero1_geometry(uint64_t n_arena, int world, int rank, uint64_t *shard_elems,
	uint64_t *shard_off, uint64_t *shard_n)
{
	uint64_t per;
	uint64_t off;

	if (world < 1 || world > ANNI_MAX_PEERS || rank < 0 || rank >= world)
		return ANNI_E_ARG;
	per = (n_arena + (uint64_t)world - 1) / (uint64_t)world;
	per = (per + ANNI_ZERO1_SHARD_ALIGN - 1) / ANNI_ZERO1_SHARD_ALIGN * ANNI_ZERO1_SHARD_ALIGN;
	if (per == 0)
		per = ANNI_ZERO1_SHARD_ALIGN;
	off = (uint64_t)rank * per;
	if (shard_elems)
		*shard_elems = per;
	if (shard_off)
		*shard_off = off < n_arena ? off : n_arena;
	if (shard_n)
		*shard_n = off < n_arena ? (n_arena - off < per ? n_arena - off : per) : 0;
	return ANNI_OK;
}

extern "C" int anni_zero1_nccl_available(void)
{
	return nccl() ? 1 : 0;
}

extern "C" int anni_zero1_unique_id(void *id_out)
{
	const nccl_api *n = nccl();

	if (!id_out)
		return ANNI_E_ARG;
	if (!n)
		return ANNI_E_CUDA;
	return n->get_unique_id((nccl_uid *)id_out) == 0 ? ANNI_OK : ANNI_E_CUDA;
}

extern "C" int anni_zero1_comm_init(const void *id, int rank, int world, void **comm_out)
{
	const nccl_api *n = nccl();
	nccl_uid uid;

	if (!id || !comm_out || world < 1 || rank < 0 || rank >= world)
		return ANNI_E_ARG;
	*comm_out = NULL;
	if (!n)
		return ANNI_E_CUDA;
	memcpy(&uid, id, sizeof(uid));
	return n->comm_init_rank(comm_out, world, uid, rank) == 0 ? ANNI_OK : ANNI_E_CUDA;
}

extern "C" void anni_zero1_comm_free(void *comm)
{
	const nccl_api *n = nccl();

	if (comm && n)
		(void)n->comm_destroy(comm);
}

static int attach(anni_zero1 *z, const void *const *peer_grad, const void *mc_grad)
{
	int rc;

	rc = anni_optstep_set_grad_arena(z->eng, z->world > 1 ? z->grad_arena : NULL, z->per, z->world);
	if (rc != ANNI_OK || !z->peer)
		return rc;
	rc = anni_optstep_set_peers(z->eng, peer_grad, z->peer_twin, z->has_fp8 ? z->peer_twin8 : NULL,
	    z->world, (uint64_t)z->rank * z->per);
	if (rc != ANNI_OK)
		return rc;
	/* remote copies first, every rank starting at another peer; this rank's own copy last */
	rc = anni_optstep_rotate_peers(z->eng, (z->rank + 1) % z->world);
	if (rc != ANNI_OK)
		return rc;
	z->mc_grad = mc_grad;
	z->mc_on = 0;
	if (mc_grad && z->mc_twin && (!z->has_fp8 || z->mc_twin8)) {
		rc = anni_optstep_set_multicast(z->eng, mc_grad, z->mc_twin, z->mc_twin8,
		    (uint64_t)z->rank * z->per);
		z->mc_on = rc == ANNI_OK;
	}
	return rc;
}

extern "C" int anni_zero1_create(const anni_zero1_config *cfg, anni_zero1 **out)
{
	anni_optstep_config ec;
	anni_zero1 *z;
	int has_fp8 = 0;
	int rc;
	int k;

	if (!out)
		return ANNI_E_ARG;
	*out = NULL;
	/* everything that can be judged without a device or a communicator comes first */
	if (!cfg || cfg->world < 1 || cfg->world > ANNI_MAX_PEERS || cfg->rank < 0 || cfg->rank >= cfg->world)
		return ANNI_E_ARG;
	if (cfg->n_seg < 0 || (cfg->n_seg > 0 && (!cfg->seg_off || !cfg->seg_flags)))
		return ANNI_E_ARG;
	if ((cfg->grad_dtype != ANNI_DT_F32 && cfg->grad_dtype != ANNI_DT_BF16)
	    || (cfg->state_dtype != ANNI_DT_F32 && cfg->state_dtype != ANNI_DT_BF16))
		return ANNI_E_ARG;
	for (k = 0; k < cfg->n_seg; k++)
		if (cfg->seg_flags[k] & ANNI_SEG_TWIN_FP8)
			has_fp8 = 1;
	if (!cfg->grad_arena || !cfg->twin_arena || (has_fp8 && !cfg->twin_fp8_arena))
		return ANNI_E_ARG;
	if (cfg->world > 1 && !cfg->nccl_comm)
		return ANNI_E_ARG;
	if (cfg->peer_grad) {
		if (!cfg->peer_twin || (has_fp8 && !cfg->peer_twin_fp8))
			return ANNI_E_ARG;
		for (k = 0; k < cfg->world; k++)
			if (!cfg->peer_grad[k] || !cfg->peer_twin[k] || (has_fp8 && !cfg->peer_twin_fp8[k]))
				return ANNI_E_ARG;
		if (cfg->peer_grad[cfg->rank] != cfg->grad_arena || cfg->peer_twin[cfg->rank] != cfg->twin_arena)
			return ANNI_E_ARG;
	}
	if (cfg->world > 1 && !nccl())
		return ANNI_E_CUDA;
	z = (anni_zero1 *)calloc(1, sizeof(*z));
	if (!z)
		return ANNI_E_NOMEM;
	z->comm = cfg->nccl_comm;
	z->rank = cfg->rank;
	z->world = cfg->world;
	z->grad_dtype = cfg->grad_dtype;
	z->n_seg = cfg->n_seg > 0 ? cfg->n_seg : 1;
	z->has_fp8 = has_fp8;
	z->peer = cfg->peer_grad != NULL && cfg->world > 1;
	z->grad_arena = cfg->grad_arena;
	z->twin_arena = cfg->twin_arena;
	z->twin_fp8_arena = cfg->twin_fp8_arena;
	z->mc_twin = cfg->mc_twin;
	z->mc_twin8 = cfg->mc_twin_fp8;
	{
		const char *e = getenv("ANNI_B200_REDUCE_CLEARS_OWN");	/* 0: the update clears every part (tuning) */

		z->clear_own = !(e && atoi(e) == 0);
	}
	(void)anni_zero1_geometry(cfg->n_arena, cfg->world, cfg->rank, &z->per, &z->shard_off, &z->shard_n);
	memset(&ec, 0, sizeof(ec));
	ec.n_arena = cfg->n_arena;
	ec.shard_off = z->shard_off;
	ec.shard_n = z->shard_n;
	ec.grad_dtype = cfg->grad_dtype;
	ec.state_dtype = cfg->state_dtype;
	ec.n_seg = cfg->n_seg;
	ec.seg_off = cfg->seg_off;
	ec.seg_flags = cfg->seg_flags;
	rc = anni_optstep_create(&ec, &z->eng);
	if (rc == ANNI_OK && cudaMalloc((void **)&z->d_tick, sizeof(float)) != cudaSuccess)
		rc = ANNI_E_NOMEM;
	if (rc == ANNI_OK && cudaMemset(z->d_tick, 0, sizeof(float)) != cudaSuccess)
		rc = ANNI_E_CUDA;
	if (rc != ANNI_OK) {
		anni_zero1_destroy(z);
		return rc;
	}
	if (z->peer)
		for (k = 0; k < z->world; k++) {
			z->peer_twin[k] = cfg->peer_twin[k];
			z->peer_twin8[k] = has_fp8 ? cfg->peer_twin_fp8[k] : NULL;
		}
	if (z->world > 1 || z->peer) {
		rc = attach(z, cfg->peer_grad, cfg->mc_grad);
		if (rc != ANNI_OK) {
			anni_zero1_destroy(z);
			return rc;
		}
	}
	*out = z;
	return ANNI_OK;
}

extern "C" void anni_zero1_destroy(anni_zero1 *z)
{
	if (!z)
		return;
	if (z->eng)
		anni_optstep_destroy(z->eng);
	cudaFree(z->d_tick);
	free(z);
}

extern "C" anni_optstep *anni_zero1_engine(anni_zero1 *z)
{
	return z ? z->eng : NULL;
}

extern "C" int anni_zero1_bind(anni_zero1 *z, float *master, void *m, void *v, void *grad_shard)
{
	anni_optstep_buffers b;
	const uint64_t base = z ? (uint64_t)z->rank * z->per : 0;
	int rc;

	if (!z || !grad_shard)
		return ANNI_E_ARG;
	memset(&b, 0, sizeof(b));
	b.master = master;
	b.m = m;
	b.v = v;
	/* one rank: the reduce-scatter is the identity, the arena itself is stepped (and cleared) */
	b.grad = z->world == 1 ? z->grad_arena : grad_shard;
	b.twin_bf16 = (uint16_t *)z->twin_arena + base;
	b.twin_fp8 = z->twin_fp8_arena ? (uint8_t *)z->twin_fp8_arena + base : NULL;
	rc = anni_optstep_bind(z->eng, &b);
	if (rc == ANNI_OK) {
		z->grad_shard = grad_shard;
		z->bufs = b;
		z->bound = 1;
	}
	return rc;
}

extern "C" int anni_zero1_set_grad_arena(anni_zero1 *z, void *grad_arena, const void *const *peer_grad,
	const void *mc_grad)
{
	if (!z || !grad_arena || (z->peer && (!peer_grad || peer_grad[z->rank] != grad_arena)))
		return ANNI_E_ARG;
	z->grad_arena = grad_arena;
	if (z->world == 1) {
		/* one rank: the engine steps the arena in place, so the arena is what it is bound to */
		if (!z->bound)
			return ANNI_OK;
		z->bufs.grad = grad_arena;
		return anni_optstep_bind(z->eng, &z->bufs);
	}
	return attach(z, peer_grad, mc_grad);
}

static int tick(anni_zero1 *z, cudaStream_t st)
{
	return nccl()->all_reduce(z->d_tick, z->d_tick, 1, NCCL_FLOAT32, NCCL_SUM, z->comm, st) == 0
	    ? ANNI_OK : ANNI_E_CUDA;
}

static int mark(void *const *events, int k, cudaStream_t st)
{
	if (!events || !events[k])
		return ANNI_OK;
	return cudaEventRecord((cudaEvent_t)events[k], st) == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}

#define TRY(call)	do { rc = (call); if (rc != ANNI_OK) return rc; } while (0)

extern "C" int anni_zero1_step(anni_zero1 *z, const anni_optstep_hyper *hp, int flags, void *stream,
	void *const *phase_events)
{
	cudaStream_t st = (cudaStream_t)stream;
	const nccl_api *n;
	const int gtype = z && z->grad_dtype == ANNI_DT_BF16 ? NCCL_BFLOAT16 : NCCL_FLOAT32;
	anni_optstep_hyper own;
	int rc;

	if (!z || !hp || !z->bound)
		return ANNI_E_ARG;
	if (z->world == 1) {
		TRY(anni_optstep_step(z->eng, hp, stream));
		for (int k = 0; k < 4; k++)
			TRY(mark(phase_events, k, st));
		return ANNI_OK;
	}
	n = nccl();
	if (!n)
		return ANNI_E_CUDA;
	if (z->peer) {
		if (!(flags & ANNI_ZERO1_GRADS_COMPLETE))
			TRY(tick(z, st));
		/* nobody else reads this rank's own part of its arena: cleared while the links are the bound */
		if (z->clear_own && !z->mc_on && (hp->flags & ANNI_STEP_ZERO_GRAD)) {
			own = *hp;
			own.flags |= ANNI_STEP_REDUCE_CLEARS_OWN;
			hp = &own;
		}
		TRY(anni_optstep_reduce_norm(z->eng, hp, stream));
	} else {
		if (n->reduce_scatter(z->grad_arena, z->grad_shard, (size_t)z->per, gtype, NCCL_SUM, z->comm, st) != 0)
			return ANNI_E_CUDA;
		TRY(anni_optstep_norm(z->eng, hp, stream));
	}
	TRY(mark(phase_events, 0, st));
	/* the sum of squares of all shards; its arrival also says that every rank has read this arena */
	if (n->all_reduce(anni_optstep_reduce_buffer(z->eng), anni_optstep_reduce_buffer(z->eng), 2,
	    NCCL_FLOAT64, NCCL_SUM, z->comm, st) != 0)
		return ANNI_E_CUDA;
	TRY(mark(phase_events, 1, st));
	TRY(anni_optstep_update(z->eng, hp, stream));
	if (z->has_fp8) {
		if (n->all_reduce(anni_optstep_amax_buffer(z->eng), anni_optstep_amax_buffer(z->eng),
		    (size_t)z->n_seg, NCCL_FLOAT32, NCCL_MAX, z->comm, st) != 0)
			return ANNI_E_CUDA;
		TRY(anni_optstep_quantize(z->eng, stream));
	}
	if (!z->peer) {
		const uint64_t base = (uint64_t)z->rank * z->per;

		if (n->all_gather((uint16_t *)z->twin_arena + base, z->twin_arena, (size_t)z->per, NCCL_BFLOAT16,
		    z->comm, st) != 0)
			return ANNI_E_CUDA;
		if (z->has_fp8 && n->all_gather((uint8_t *)z->twin_fp8_arena + base, z->twin_fp8_arena,
		    (size_t)z->per, NCCL_UINT8, z->comm, st) != 0)
			return ANNI_E_CUDA;
	}
	TRY(mark(phase_events, 2, st));
	if (z->peer)
		TRY(tick(z, st));	/* every rank's twins have landed in every arena */
	TRY(mark(phase_events, 3, st));
	return ANNI_OK;
}
