/*
** ZeRO-1 step for a C trainer: the optimizer state of one packed arena sharded over the GPUs
** of one node, one process per GPU, NCCL for the small exchanges.
**
** No counterpart in the reference: its trainer is single-GPU (its README lists multi-GPU as
** open); the call a multi-GPU build of it would make sits where lang/lm_train.c:1349-1351
** calls lm_adam_step_scaled today.  Per step, on every rank, one call:
**
**     anni_zero1_step(z, &hp, flags, stream, NULL);
**
** which queues, on `stream`:
**   peer mode (the caller handed in peer-accessible pointers of every rank's arenas, e.g. from
**   CUDA IPC or symmetric memory):
**     [all-reduce of one float: every rank's gradients are complete]
**     reduce-scatter + norm kernel   reads this shard out of every rank's gradient arena and
**                                    clears the part of this rank's arena that only it reads
**     all-reduce(sum) of 2 doubles   global sum of squares and non-finite flag
**     update kernel                  decision, AdamW, twins stored into every rank's twin arena,
**                                    the rest of this rank's gradient arena cleared
**     [all-reduce(max) of per-tensor amax; quantise kernel]       (e4m3 twins only)
**     all-reduce of one float        every rank's twins have landed
**   NCCL mode (no peer pointers):
**     ncclReduceScatter(sum) of the gradient arena into the shard buffer, norm kernel, the same
**     all-reduce, update kernel, [amax all-reduce, quantise kernel], ncclAllGather of the twins
**     in place inside the twin arena.
**
** Layout: the arena of n_arena elements is padded to world * shard elements (shard a multiple
** of 4096, see anni_zero1_geometry) and cut into equal contiguous shards irrespective of tensor
** boundaries; rank r owns master / m / v of shard r, and holds a full gradient arena (input) and
** a full twin arena (output).
**
** NCCL is resolved at run time (dlopen of libnccl.so.2, preferring the copy already loaded in
** the process), so the library itself loads on machines without it.
*/
#ifndef ANNI_ZERO1_H__
#define ANNI_ZERO1_H__

#include <stddef.h>
#include <stdint.h>
#include "anni_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct anni_zero1 anni_zero1;

#define ANNI_ZERO1_UNIQUE_ID_BYTES	128	/* sizeof(ncclUniqueId) */
#define ANNI_ZERO1_SHARD_ALIGN		4096	/* elements: every shard base stays 16-byte aligned for all types */

/* anni_zero1_step flags */
#define ANNI_ZERO1_GRADS_COMPLETE	1	/* every rank's gradients were complete before the previous
						** step's closing exchange: skip the opening one (peer mode) */

typedef struct anni_zero1_config {
	uint64_t	n_arena;	/* elements of the unpadded arena */
	int		grad_dtype;	/* ANNI_DT_* */
	int		state_dtype;
	int		n_seg;		/* tensor table as in anni_optstep_config (host arrays, copied) */
	const int64_t	*seg_off;
	const uint32_t	*seg_flags;
	int		rank;
	int		world;		/* 1 .. 8 */
	void		*nccl_comm;	/* ncclComm_t over the `world` ranks; stays the caller's */
	/* this rank's own arenas, world * shard elements each (twin_fp8_arena NULL without e4m3 twins) */
	void		*grad_arena;
	void		*twin_arena;
	void		*twin_fp8_arena;
	/*
	** peer mode: every rank's arenas as seen from THIS process, `world` entries each, entry
	** `rank` being the arenas above.  NULL: NCCL mode.
	*/
	const void *const	*peer_grad;
	void *const		*peer_twin;
	void *const		*peer_twin_fp8;
	/* optional NVSwitch multicast addresses of the same three arenas (peer mode), or NULL */
	const void	*mc_grad;
	void		*mc_twin;
	void		*mc_twin_fp8;
} anni_zero1_config;

/*
** Shard geometry: elements per shard including padding, and what `rank` owns of the unpadded
** arena (shard_n may be 0 for the last ranks of a tiny arena).  Pure arithmetic.
*/
int	anni_zero1_geometry(uint64_t n_arena, int world, int rank, uint64_t *shard_elems,
		uint64_t *shard_off, uint64_t *shard_n);

/* 1 when libnccl.so.2 and the entry points used here could be resolved, else 0. */
int	anni_zero1_nccl_available(void);
/*
** Convenience for callers without a communicator of their own: rank 0 calls
** anni_zero1_unique_id, ships the 128 bytes to the other ranks by any means, every rank calls
** anni_zero1_comm_init (collective; the current CUDA device is the rank's).  anni_zero1_comm_free
** destroys such a communicator.
*/
int	anni_zero1_unique_id(void *id_out);
int	anni_zero1_comm_init(const void *id, int rank, int world, void **comm_out);
void	anni_zero1_comm_free(void *comm);

/*
** Creates the rank's engine on the current device (arguments are checked before any device or
** NCCL call: ANNI_E_ARG for a bad table, rank, world or a missing arena; world > 1 needs
** nccl_comm).  bind names the shard buffers (shard elements each; grad_shard is where the
** reduced gradients land: scratch between steps).
*/
int	anni_zero1_create(const anni_zero1_config *cfg, anni_zero1 **out);
int	anni_zero1_bind(anni_zero1 *z, float *master, void *m, void *v, void *grad_shard);
/* Another set of gradient arenas (e.g. one per micro-step buffer) for the following steps. */
int	anni_zero1_set_grad_arena(anni_zero1 *z, void *grad_arena, const void *const *peer_grad,
		const void *mc_grad);
/*
** One sharded step, queued on `stream`.  phase_events: NULL, or four cudaEvent_t handles that
** are recorded after the reduce-scatter + norm, after the all-reduce, after the update (and
** quantise, and in NCCL mode the all-gather), and after the closing exchange.
*/
int	anni_zero1_step(anni_zero1 *z, const anni_optstep_hyper *hp, int flags, void *stream,
		void *const *phase_events);
/* The shard's engine, for status, loss scale and the small device buffers. */
anni_optstep	*anni_zero1_engine(anni_zero1 *z);
void	anni_zero1_destroy(anni_zero1 *z);

#ifdef __cplusplus
}
#endif

#endif
