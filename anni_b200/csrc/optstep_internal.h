/*
** Internal interface between the packed-arena engine (optstep.cu) and the
** reference-compatible device API (gpu_compat.cu).  Not installed.
*/
#ifndef ANNI_OPTSTEP_INTERNAL_H__
#define ANNI_OPTSTEP_INTERNAL_H__

#include <cuda_runtime.h>
#include <stdint.h>
#include "anni_b200.h"

#define ANNI_THREADS		256	/* threads per block of every arena kernel */
#define ANNI_VEC		8	/* elements per thread per chunk, norm phase (16-byte loads of bf16) */
#define ANNI_CHUNK		(ANNI_THREADS * ANNI_VEC)
#define ANNI_CHUNK_LOG2		11
/*
** Update and quantise phases: four elements per thread per chunk.  Measured on B200 with
** the update's access mix (4 read and 5 write streams, 22 bytes per element): HBM
** throughput peaks with about 36 KB of loads queued per SM and drops 5-8 % with 48-72 KB,
** while the arithmetic wants 1024 threads per SM to hide its latencies -- hence 4 blocks x
** 256 threads x 4 elements for bf16 moments (12 bytes per element in flight), 3 blocks for
** fp32 moments (14-16 bytes).
*/
#define ANNI_UVEC		4
#define ANNI_UCHUNK		(ANNI_THREADS * ANNI_UVEC)
#define ANNI_UCHUNK_LOG2	10
#ifndef ANNI_PIPE_LAG
#define ANNI_PIPE_LAG		2	/* default of anni_launch.pipe_lag */
#endif
/* tile of the transposed e4m3 twins: rows x columns of the master (kernel and host tile count) */
#define ANNI_TT_R		128
#define ANNI_TT_C		64
#define ANNI_MAX_BLOCKS		2048	/* capacity of the per-block partial table */
#define ANNI_MAX_PEERS		8	/* GPUs of one NVSwitch domain */
/* polls of a bounded device wait before it gives up (each poll sleeps >= 32 ns) */
#define ANNI_WAIT_POLLS		(1u << 23)

/*
** Device-resident control block of one engine (or of the legacy entry points).
** Everything the kernels exchange besides the big buffers lives here.
*/
typedef struct anni_control {
	double		reduce[2];	/* {sum of squares, non-finite count}; all-reduced by ZeRO-1 callers */
	double		norm;
	double		eff_scale;
	double		loss_scale;	/* <= 0: state machine off */
	double		ls_growth;
	double		ls_backoff;
	double		ls_min;
	double		ls_max;
	int32_t		ls_interval;
	int32_t		good_steps;
	int32_t		skipped;
	int32_t		error;
	int32_t		steps_done;
	uint32_t	bar_count;	/* arrivals at the in-kernel barriers; reset by the last block */
	uint32_t	norm_ticket;	/* blocks that finished the norm kernel */
	uint32_t	done_ticket;	/* blocks that finished the update */
	uint32_t	pipe_polls;	/* polls spent waiting for other blocks' tensors (one-launch fp8 step) */
	double		partials[ANNI_MAX_BLOCKS];
} anni_control;

/* Arguments of one launch, passed by value. */
typedef struct anni_launch {
	float		*master;
	void		*m;
	void		*v;
	void		*grad;
	uint16_t	*twin16;
	uint8_t		*twin8;
	uint64_t	n;		/* shard elements */
	uint64_t	arena_off;	/* arena coordinate of shard element 0 */
	const int64_t	*seg_off;	/* device, n_seg + 1 */
	const uint32_t	*seg_flags;	/* device, n_seg */
	float		*seg_amax;	/* device, n_seg */
	float		*seg_scale;	/* device, n_seg */
	uint32_t	*seg_done;	/* device, n_seg: blocks that have finished updating each tensor (one-launch fp8 step) */
	const anni_seg_derived *seg_aux;	/* device, n_seg, or NULL: shapes and targets of the derived twins */
	uint16_t	*qkv_packed;	/* [Wq|Wk|Wv] bf16 matrices, one per layer */
	uint8_t		*fp8_t;		/* transposed e4m3 twins */
	int		n_seg;
	int		flags;		/* ANNI_STEP_* | ANNI_LAUNCH_* */
	int		aligned;	/* every buffer 16-byte aligned: vector path allowed */
	int		sc_log2;	/* log2 of the chunks per super-chunk (see walk_chunk) */
	int		pipe_lag;	/* one-launch fp8 step: quantising trips per round while tensors queue up (else one) */
	double		grad_scale;
	double		clip;
	double		b1;
	double		omb1;
	double		b2;
	double		omb2;
	double		lrbc1d;		/* the same three in double */
	double		ibc2d;
	double		epsd;
	double		lrwdd;		/* lr * weight_decay */
	float		lrbc1;		/* lr / (1 - beta1^t) */
	float		ibc2;		/* 1 / (1 - beta2^t) */
	float		ibc2_s24;	/* ibc2 * 2^24, eps * 2^40, lrbc1 * 2^40: see adam_elem */
	float		eps_s40;
	float		lrbc1_s40;
	float		eps;
	float		lrwd;		/* lr * weight_decay */
	/*
	** ZeRO-1 over peer memory (all NULL / 0 on one GPU).  peer_grad[k]: rank k's
	** copy of THIS shard's gradients (its full gradient arena + this shard's
	** offset), read by the fused reduce-scatter + norm kernel.  twin_peer[k]:
	** where THIS shard's bf16 twins go inside rank k's full twin arena (this
	** rank included), written by the update phase in place of an all-gather.
	*/
	const void	*peer_grad[ANNI_MAX_PEERS];
	uint16_t	*twin_peer[ANNI_MAX_PEERS];
	uint8_t		*twin8_peer[ANNI_MAX_PEERS];
	int		n_peers;	/* world size when peer memory is in use, else 0 */
	/*
	** NVSwitch multicast addresses of the same arenas at this shard's offset (NULL: not in use).
	** mc_grad: multimem.ld_reduce returns the sum over all ranks' copies, reduced in the switch;
	** mc_twin / mc_twin8: multimem.st lands in every rank's copy.
	*/
	const void	*mc_grad;
	uint16_t	*mc_twin;
	uint8_t		*mc_twin8;
	/*
	** ZeRO-1, "the step leaves the gradients zeroed" (lang/lm_adam.c:597 of the reference): the
	** buffer the backward pass accumulates into is this rank's FULL gradient arena, of which the
	** update only ever sees the reduced shard.  zero_base = the arena at the element that stands
	** for shard element 0 of part 0, zero_stride = elements per part, zero_parts = parts (world
	** size): the update then clears element e of every part where it would have cleared
	** grad[e].  NULL / 0: clear the bound gradient buffer itself (one GPU).
	*/
	void		*zero_base;
	uint64_t	zero_stride;
	int		zero_parts;
	/*
	** Peer-memory ZeRO-1: this rank's own part of its arena is read by nobody else, so the
	** reduce can clear it as it reads it, while the links rather than local memory bound that
	** kernel.  own_clear = that part at shard element 0 (reduce: clear what was read; NULL: leave
	** it), zero_done = 1 + the index of a part the update need not clear any more (0: none).
	*/
	void		*own_clear;
	int		zero_done;
	anni_control	*ctl;
} anni_launch;

/* launch flags beyond ANNI_STEP_* */
#define ANNI_LAUNCH_HOST_COEF	0x100	/* grad_scale is final: no norm, no decision (legacy two-call sequence) */
#define ANNI_LAUNCH_NEED_NORM	0x200	/* the norm feeds a clip or a finite check */
#define ANNI_LAUNCH_HAS_FP8	0x400	/* some segment asks for an e4m3 twin */
#define ANNI_LAUNCH_ACCUMULATE	0x800	/* norm over a part of the shard: add to the running sum */
#define ANNI_LAUNCH_NO_EPILOGUE	0x1000	/* update over a part of the shard that is not the last: the step stays open */
#define ANNI_LAUNCH_PIPE_STREAM	0x4000	/* ... and store those tensors' masters with the streaming hint all the same (tuning) */
#define ANNI_LAUNCH_FP8_PIPE	0x2000	/* one-launch step: quantise tensor by tensor behind the update (see update_phase) */

#ifdef __cplusplus
extern "C" {
#endif

/*
** Kernel launchers (optstep.cu).  `blocks` is the resident grid (anni_grid_blocks, at most
** ANNI_MAX_BLOCKS); norm / update / fused may launch fewer, the same number for the same
** dtypes and step flags, so the two forms of the step share their block partials.
*/
int	anni_launch_norm(const anni_launch *a, int grad_dtype, int state_dtype, int blocks, cudaStream_t st);
int	anni_launch_update(const anni_launch *a, int grad_dtype, int state_dtype, int blocks,
		cudaStream_t st);
int	anni_launch_fused(const anni_launch *a, int grad_dtype, int state_dtype, int blocks,
		cudaStream_t st);
int	anni_launch_quantize(const anni_launch *a, int blocks, cudaStream_t st);
int	anni_launch_quantize_transposed(const anni_launch *a, const int64_t *tile_prefix, int64_t n_tiles,
		int blocks, cudaStream_t st);
int	anni_launch_barrier_timeout(anni_control *ctl, int blocks, unsigned max_polls, cudaStream_t st);
int	anni_launch_reduce_norm(const anni_launch *a, int grad_dtype, int blocks, cudaStream_t st);
/* clears elements [from, stride) of every part of a gradient arena (see anni_launch.zero_base) */
int	anni_launch_zero_tail(void *arena, int grad_dtype, uint64_t from, uint64_t stride, int parts,
		cudaStream_t st);
int	anni_launch_f32_to_bf16(uint16_t *dst, const float *src, uint64_t n, cudaStream_t st);
int	anni_launch_axpy(float *y, const float *x, float a, uint64_t n, cudaStream_t st);
/* Persistent-grid size for the given kernel family on the current device. */
int	anni_grid_blocks(int grad_dtype, int state_dtype, int cooperative);
/* Grid and super-chunk size every launcher of the step kernels uses (tuning knobs applied). */
int	anni_engine_geometry(int grad_dtype, int state_dtype, int *blocks, int *sc_log2);
/* Fills the hyper-parameter part of a launch; ANNI_E_ARG on values the reference rejects. */
int	anni_fill_hyper(anni_launch *a, const anni_optstep_hyper *hp);
void	anni_count_launch(void);

/* ANN_OP_PROF event pairs (gpu_compat.cu): begin returns a slot (or -1: profiling off), end closes it */
enum { ANNI_OP_ADAM, ANNI_OP_SUMSQ, ANNI_OP_COLSUM, ANNI_OP_AXPY, ANNI_OP_CONVERT, ANNI_OP_N };
int	anni_op_begin(int op, void *stream);
void	anni_op_end(int slot, void *stream);
/* host gradient vector -> its slice of a device gradient flat (see gpu_mat_col_sum_add) */
int	anni_colsum_register(const float *host, float *dev, int cols);
void	anni_colsum_forget(const void *dev_lo, const void *dev_hi);

#ifdef __cplusplus
}
#endif

#endif
