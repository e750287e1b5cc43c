/*
** anni_b200 -- B200 (sm_100a) optimizer-step engine for AnnI's decoder-only LM
** trainer.  C ABI: plain pointers and sizes, no C++ or framework types.
**
** Two groups of entry points live in libanni_b200.so:
**
**  1. anni_optstep_*  (this header): the packed-arena engine.  One engine owns
**     one contiguous shard of the flat parameter arena (the whole arena on one
**     GPU, 1/N of it under ZeRO-1) and runs the step as a fused pass: global
**     gradient-norm reduction, unscale + non-finite skip decision, AdamW with
**     decoupled weight decay, fp32 master write, fp32 or bf16 moments, bf16 /
**     fp8-e4m3 weight twins with per-tensor amax.  Every decision is taken on
**     the device; the host never waits inside a step.
**
**  2. the reference's own device API (num/gpu.h of the reference project),
**     declared in anni_gpu_compat.h: the ~20 symbols its optimizer calls get
**     real bodies on top of the same kernels, the rest answer -1 / NULL like
**     the reference's stub backend, so its trainer links unchanged.
**
** Error convention (that of num/gpu.h:78-80,134-139): int functions return 0
** when the work was queued on the device and a negative value when nothing was
** done.  There is no CPU fallback inside this library.
*/
#ifndef ANNI_B200_H__
#define ANNI_B200_H__

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of the gradient and moment buffers */
#define ANNI_DT_F32	0
#define ANNI_DT_BF16	1

/* per-segment flags */
#define ANNI_SEG_WD		1u	/* decoupled weight decay applies to this tensor */
#define ANNI_SEG_TWIN_BF16	2u	/* emit a bf16 twin (round to nearest even) */
#define ANNI_SEG_TWIN_FP8	4u	/* emit an e4m3 twin with a per-tensor scale */

/* per-step flags */
#define ANNI_STEP_CHECK_FINITE	1	/* skip the step when the norm is not finite */
#define ANNI_STEP_ZERO_GRAD	2	/* leave the gradient shard zeroed, as the reference step does */
#define ANNI_STEP_DEV_LOSS_SCALE 4	/* divide grad_scale by the device-resident loss scale */
/*
** Evaluate the parameter update lr*(m/bc1)/(sqrt(v/bc2)+eps) in double (the
** reference's own expression, lang/lm_adam.c:592-593 of the reference) instead of
** in float with SFU square root and reciprocal: the master then equals the
** reference's float in all but ~1e-7 of the elements, at about 7 % more time.
*/
#define ANNI_STEP_EXACT_UPDATE	8
/*
** ZeRO-1 over peer memory, with a gradient arena named (anni_optstep_set_grad_arena) and
** ANNI_STEP_ZERO_GRAD set: anni_optstep_reduce_norm[_range] clears this rank's own part of its
** arena as it reads it (no other rank reads that part), and anni_optstep_update[_range] of the
** same step, given the same flag, clears the other parts only.  Not with multicast reduction.
** Both calls answer ANNI_E_ARG when the arena or the own part cannot be told from the peers.
*/
#define ANNI_STEP_REDUCE_CLEARS_OWN	16

/* error codes (negative return values; also anni_optstep_status.error) */
#define ANNI_OK			0
#define ANNI_E_ARG		(-1)	/* bad argument: nothing was launched */
#define ANNI_E_CUDA		(-2)	/* a CUDA runtime call failed */
#define ANNI_E_BARRIER_TIMEOUT	(-3)	/* a bounded device-side wait gave up; state untouched by late blocks */
#define ANNI_E_NOMEM		(-4)
#define ANNI_E_LIMIT		(-5)	/* size beyond a stated maximum */

typedef struct anni_optstep anni_optstep;

/*
** Shape of one engine.  The arena is the reference's flat layout
** (lang/lm_adam.c:217-311: one running element offset per tensor, unpadded, the
** bf16 twin at the same element offset as the fp32 master, num/gpu_cuda.cu:
** 2026-2034).  seg_off has n_seg + 1 ascending ARENA element offsets
** (seg_off[0] = 0, seg_off[n_seg] = n_arena); both arrays are host memory and
** are copied.  n_seg = 0 means one segment covering everything with
** ANNI_SEG_WD | ANNI_SEG_TWIN_BF16, which is what the reference's flat kernels
** do (num/gpu_cuda.cu:8557-8580).
*/
typedef struct anni_optstep_config {
	uint64_t	n_arena;	/* elements in the whole arena */
	uint64_t	shard_off;	/* first arena element this engine owns */
	uint64_t	shard_n;	/* elements this engine owns (may be 0) */
	int		grad_dtype;	/* ANNI_DT_* */
	int		state_dtype;	/* ANNI_DT_*: storage of m and v */
	int		n_seg;
	const int64_t	*seg_off;
	const uint32_t	*seg_flags;
} anni_optstep_config;

/*
** Device buffers of the shard, caller-owned, each 16-byte aligned; element i of
** every buffer is arena element shard_off + i.  twin_bf16 / twin_fp8 may be
** NULL when no segment asks for that twin.
*/
typedef struct anni_optstep_buffers {
	float	*master;	/* fp32 [shard_n], updated in place */
	void	*m;		/* state_dtype [shard_n] */
	void	*v;
	void	*grad;		/* grad_dtype [shard_n] */
	void	*twin_bf16;	/* uint16 [shard_n] */
	void	*twin_fp8;	/* uint8  [shard_n] */
} anni_optstep_buffers;

/*
** One step's scalars, named as in the reference (lang/lm_adam.h:37-53 and
** the argument list at num/gpu.h:129-132).  t is the step number AFTER the
** caller incremented it (t >= 1), exactly the `t` of gpu_adam_step_dev_bf16.
** grad_scale multiplies every gradient (1/batch, and 1/loss_scale unless the
** device-resident scale is used).  grad_clip = 0 turns clipping off.
*/
typedef struct anni_optstep_hyper {
	double	lr;
	double	beta1;
	double	beta2;
	double	eps;
	double	weight_decay;
	double	grad_clip;
	double	grad_scale;
	int	t;
	int	flags;		/* ANNI_STEP_* */
} anni_optstep_hyper;

/* What the device decided, read back on request. */
typedef struct anni_optstep_status {
	double	sumsq;		/* sum of squares of the raw gradients (all ranks once reduced) */
	double	norm;		/* sqrt(sumsq) * |effective grad scale|: the pre-clip norm (lm_adam.h:53) */
	double	eff_scale;	/* multiplier actually applied to the gradients */
	double	loss_scale;	/* device-resident loss scale after this step */
	int32_t	skipped;	/* 1: non-finite norm, parameters and moments untouched */
	int32_t	error;		/* ANNI_E_* raised on the device, 0 if none */
	int32_t	good_steps;	/* clean steps since the loss scale last changed */
	int32_t	steps_done;	/* update launches completed since creation */
} anni_optstep_status;

/* ---- life cycle ---------------------------------------------------------- */

/* Creates an engine on the current CUDA device (allocates its small control
** block and device copies of the segment table).  Every later call on the engine
** must be made with that device current (one process per GPU: set it once). */
int	anni_optstep_create(const anni_optstep_config *cfg, anni_optstep **out);
void	anni_optstep_destroy(anni_optstep *h);
int	anni_optstep_bind(anni_optstep *h, const anni_optstep_buffers *buf);

/* ---- the step -------------------------------------------------------------- */

/*
** Whole step in ONE cooperative launch on `stream` (a cudaStream_t, NULL = the
** legacy stream): norm phase, device-wide bounded barrier, decision, update
** phase, twin emission, and for fp8 segments a second barrier and the quantising
** phase (preceded by one small memset of the per-tensor amax table; with
** ANNI_B200_FP8_PIPE=1 the quantiser instead follows the update tensor by tensor
** inside the same phase and the memset goes away).  Replaces the reference sequence gpu_grad_sumsq -> host
** sqrt/clip/skip -> gpu_adam_step_dev_bf16 (lang/lm_adam.c:466-493) and its two
** host round trips.  Single-GPU form: the norm is this shard's alone.
*/
int	anni_optstep_step(anni_optstep *h, const anni_optstep_hyper *hp, void *stream);

/*
** The same step cut at its two global dependencies, for ZeRO-1: between the
** calls the caller all-reduces small device buffers across ranks.
**   anni_optstep_norm      local sum of squares -> reduce buffer {sumsq, nonfinite}
**     [all-reduce SUM of anni_optstep_reduce_buffer(h): 2 doubles]
**   anni_optstep_update    decision + AdamW + bf16 twins + per-tensor amax
**     [all-reduce MAX of anni_optstep_amax_buffer(h): n_seg floats; fp8 only]
**   anni_optstep_quantize  scale from amax, e4m3 twins of the fresh master
*/
int	anni_optstep_norm(anni_optstep *h, const anni_optstep_hyper *hp, void *stream);
int	anni_optstep_update(anni_optstep *h, const anni_optstep_hyper *hp, void *stream);
int	anni_optstep_quantize(anni_optstep *h, void *stream);
/*
** The step for a caller whose gradient PRODUCER already knows the sum of squares (the last
** epilogue of the backward pass, a reduce-scatter that squares what it writes): no norm pass, so
** the gradients are read once.  d_sumsq: device double[2] = {sum of squares of the raw gradients,
** count of non-finite values (0 if none)}, read when the stream gets there.  Otherwise identical
** to anni_optstep_step, e4m3 twins included (two launches then, the update and the quantiser).
*/
int	anni_optstep_step_with_sumsq(anni_optstep *h, const anni_optstep_hyper *hp, const double *d_sumsq,
		void *stream);
double	*anni_optstep_reduce_buffer(anni_optstep *h);	/* device double[2] */
float	*anni_optstep_amax_buffer(anni_optstep *h);	/* device float[n_seg] */
float	*anni_optstep_scale_buffer(anni_optstep *h);	/* device float[n_seg]: dequantisation scales */

/*
** Derived twins the forward pass consumes, emitted by the step instead of being rebuilt from
** the twins afterwards (in the reference: qkv_wt_pack_kernel, num/gpu_cuda.cu:6456, once per
** optimizer step and layer; f32_transpose_to_fp8_kernel, :898-924, the [N,K] layout of e4m3
** weights).  One entry per tensor of the segment table:
**   rows, cols     the matrix shape (rows * cols = tensor elements); 0, 0 for vectors
**   pack_ld        != 0: the tensor's bf16 twin is ALSO stored into `qkv_packed` as a block of a
**                  wider row-major matrix: element (r, c) at pack_off + r * pack_ld + c.  For a
**                  layer's [Wq|Wk|Wv] (D x 3D): pack_ld = 3D, pack_off = layer base + 0 / D / 2D.
**   fp8_t_off      >= 0 (tensor must carry ANNI_SEG_TWIN_FP8): its e4m3 twin is written
**                  TRANSPOSED ([cols][rows], same per-tensor scale) at this byte offset of
**                  `fp8_t` instead of row-major into twin_fp8.  -1: row-major as usual.
** Arrays are host memory and are copied; buffers are device memory owned by the caller.
** Single-GPU engines only (shard = whole arena).
*/
typedef struct anni_seg_derived {
	int32_t	rows;
	int32_t	cols;
	int64_t	pack_off;
	int32_t	pack_ld;
	int32_t	reserved;
	int64_t	fp8_t_off;
} anni_seg_derived;

int	anni_optstep_set_derived(anni_optstep *h, const anni_seg_derived *aux, void *qkv_packed,
		void *fp8_t);

/*
** ZeRO-1 over peer memory (NVLink / NVSwitch), no counterpart in the reference
** (it is single-GPU).  Instead of an NCCL reduce-scatter before and an
** all-gather after the step, the kernels themselves move the data:
**   anni_optstep_set_peers   peer_grad[k]  = rank k's FULL gradient arena (element 0 of the
**                            padded arena), peer_twin[k] / peer_twin_fp8[k] = rank k's FULL
**                            twin arenas; all peer-accessible device pointers valid in this
**                            process (e.g. CUDA IPC or symmetric memory), n_peers = world
**                            size <= 8, arena_off_padded = this shard's first element in
**                            those padded arenas.  n_peers = 0 detaches.
**   anni_optstep_reduce_norm replaces reduce-scatter + anni_optstep_norm: reads this shard from
**                            every peer's arena, sums in rank order in float, writes the
**                            reduced shard into the bound gradient buffer, leaves {sumsq,
**                            nonfinite} in the reduce buffer.  Queue it after a barrier that
**                            says every rank's gradients are complete.
**   anni_optstep_update / anni_optstep_quantize then write the twins of this shard into every
**                            peer's arena (this rank's included): queue a barrier after them
**                            before anyone reads the twins.
** The kernels contain no cross-GPU waits; ordering between ranks is the caller's (stream-ordered
** collectives or events).
*/
int	anni_optstep_set_peers(anni_optstep *h, const void *const *peer_grad, void *const *peer_twin,
		void *const *peer_twin_fp8, int n_peers, uint64_t arena_off_padded);
int	anni_optstep_reduce_norm(anni_optstep *h, const anni_optstep_hyper *hp, void *stream);
/*
** The same two calls over a PART of the shard (elements [elem_off, elem_off + elem_n) of it,
** elem_off a multiple of 4096), so that a caller can pipeline the step with its own data
** movement: e.g. copy engines pull the peers' copies of the shard into local memory part by
** part (peer_grad[k] given to anni_optstep_set_peers then points at those LOCAL copies) and push
** the locally stored twins out, each overlapping the kernel of the neighbouring part.  Measured
** on B200s this is no faster than the kernels moving the data themselves (2.78 against 2.69 ms
** per step at four ranks), so it is an option, not the default.
**   anni_optstep_reduce_norm_range  flags: ANNI_RANGE_ACCUMULATE = add this part's sum of squares
**                                   to the reduce buffer instead of replacing it (every part but
**                                   the first)
**   anni_optstep_update_range       flags: ANNI_RANGE_LAST = this part closes the step (loss-scale
**                                   state machine, step counter); ANNI_RANGE_LOCAL_TWINS = store
**                                   the twins through the bound buffers only, although peers are set;
**                                   ANNI_RANGE_FIRST = clear the per-tensor amax (fp8 twins)
**   anni_peer_copy                  one asynchronous copy between any two device addresses valid
**                                   in this process (plain cudaMemcpyAsync; the driver picks the
**                                   copy engine for peer memory)
*/
#define ANNI_RANGE_ACCUMULATE	1
#define ANNI_RANGE_LAST		2
#define ANNI_RANGE_LOCAL_TWINS	4
#define ANNI_RANGE_FIRST	8
int	anni_optstep_reduce_norm_range(anni_optstep *h, const anni_optstep_hyper *hp, uint64_t elem_off,
		uint64_t elem_n, int flags, void *stream);
int	anni_optstep_update_range(anni_optstep *h, const anni_optstep_hyper *hp, uint64_t elem_off,
		uint64_t elem_n, int flags, void *stream);
int	anni_peer_copy(void *dst, const void *src, size_t nbytes, void *stream);
/* anni_optstep_quantize with ANNI_RANGE_LOCAL_TWINS: the e4m3 twins through the bound buffer only. */
int	anni_optstep_quantize_ex(anni_optstep *h, int flags, void *stream);
/*
** Device memory with the GPU's memory compression switched on, for buffers whose contents
** compress well: the gradient arena, which every step leaves zeroed.  The L2 then writes such
** lines back to HBM at a fraction of their size.  No counterpart in the reference (its
** optimizer allocates the flats with gpu_malloc); results do not depend on it.
**   anni_arena_alloc   nbytes of zeroed memory on the current device; *mapped_bytes is what to
**                      pass to anni_arena_free.  ANNI_E_LIMIT: the device or driver does not
**                      offer compressible memory (nothing allocated: use cudaMalloc).
**   anni_arena_free    synchronises the device, unmaps and releases.
** The memory comes from the driver's virtual-memory interface: release it with anni_arena_free
** only (never cudaFree), and do not expect cudaIpcGetMemHandle to export it.
*/
int	anni_arena_alloc(size_t nbytes, void **out, size_t *mapped_bytes, int *compressed);
int	anni_arena_free(void *ptr, size_t mapped_bytes);
/*
** Optional, after anni_optstep_set_peers: NVSwitch multicast addresses of the same three arenas
** (element 0 of the padded arena; NULL for any that has none).  The reduce kernel then issues one
** multimem.ld_reduce per vector (the switch adds all ranks' copies; bf16 accumulated in float) and
** the update / quantise phases one multimem.st per vector (the switch replicates it into every
** rank's arena) instead of N peer loads / stores: each GPU's link carries its own shard once in
** the light direction.  A later anni_optstep_set_peers clears them.
*/
int	anni_optstep_set_multicast(anni_optstep *h, const void *mc_grad, void *mc_twin,
		void *mc_twin_fp8, uint64_t arena_off_padded);

/*
** Order in which the peers set by anni_optstep_set_peers are visited: `first` (an index into those
** arrays) comes first, the others follow cyclically.  Give every rank a different start --
** (rank + 1) % n_peers puts the remote copies first and the rank's own last -- so that at any
** moment the ranks pull from, and store to, different peers instead of all starting at rank 0.
** The reduce kernel adds the copies in that order (float addition: the result is the same on
** every run, but differs in the last bit from another order unless the sum is exact).
*/
int	anni_optstep_rotate_peers(anni_optstep *h, int first);
/*
** ZeRO-1 and "the step leaves the gradients zeroed" (lang/lm_adam.c:597, num/gpu.h:125-127 of the
** reference; its trainer relies on it, lang/lm_train.c:1220-1226): the buffer the backward pass
** accumulates into is this rank's FULL gradient arena, not the reduced shard the update works on.
** Name that arena here (`arena` = its element 0, `parts` shards of `stride` elements each, stride
** a multiple of 8 and >= this engine's shard) and anni_optstep_update / _update_range with
** ANNI_STEP_ZERO_GRAD clear the whole arena -- element e of every part where they would have
** cleared the bound gradient buffer, plus the ends of the parts beyond this shard's length --
** instead of that buffer.  Queue the update after every peer has read the arena (the all-reduce
** of the reduce buffer says so).  arena = NULL: back to clearing the bound buffer.
*/
int	anni_optstep_set_grad_arena(anni_optstep *h, void *arena, uint64_t stride, int parts);

/* Blocks until `stream` has finished the queued steps, then copies the status. */
int	anni_optstep_status_read(anni_optstep *h, anni_optstep_status *out, void *stream);

/*
** Dynamic loss scale kept on the device: a skipped step multiplies it by
** `backoff`, `growth_interval` clean steps in a row multiply it by `growth`.
** Steps that pass ANNI_STEP_DEV_LOSS_SCALE use grad_scale / loss_scale.  The
** reference has no counterpart (its fp16 loss scaling was removed); scale <= 0
** switches the state machine off.
*/
int	anni_optstep_loss_scale_init(anni_optstep *h, double scale, int growth_interval,
		double growth, double backoff, double min_scale, double max_scale);

/*
** The whole step (same kernel and arithmetic as anni_optstep_step) for callers
** that cannot allocate device memory: no engine is created, and the working
** memory the step needs (barrier counters, per-block partial sums, the device
** copy of the tensor table, per-tensor amax/scale) is a fixed array built into
** the library, present on every GPU that loads it.  No counterpart in the
** reference.  Limits and rules:
**   - at most ANNI_NOALLOC_MAX_SEG tensors in cfg->seg_off / seg_flags; more is
**     refused with ANNI_E_LIMIT before anything is queued;
**   - all calls on one device share that array: queue them one after another on
**     a single stream; calls that overlap on the GPU corrupt each other;
**   - the first call on a device resolves the array's device address: make it
**     during start-up, before any stream capture on that device;
**   - ANNI_STEP_DEV_LOSS_SCALE is not available (fold 1/loss_scale into grad_scale);
**   - cfg->seg_off / seg_flags are copied from host memory by every call: keep them valid until
**     the call returns; a stream in capture mode is refused with ANNI_E_ARG.
** cfg, buf, hp as for create / bind / step.  seg_scale_out (device, n_seg floats,
** may be NULL) receives the e4m3 dequantisation scales when fp8 twins are asked for.
*/
#define ANNI_NOALLOC_MAX_SEG	1024
int	anni_optstep_step_noalloc(const anni_optstep_config *cfg, const anni_optstep_buffers *buf,
		const anni_optstep_hyper *hp, float *seg_scale_out, void *stream);
/* Status of the last no-alloc step on the current device (synchronises `stream`). */
int	anni_optstep_status_noalloc(anni_optstep_status *out, void *stream);

/*
** Failure-path self-test of the bounded device wait: launches the engine's grid against a
** barrier that expects one block more than exists, with a poll limit of `max_polls` (keep it
** small: 65536 polls is a few milliseconds).  Every block gives up, nothing faults or hangs;
** afterwards anni_optstep_status_read reports error == ANNI_E_BARRIER_TIMEOUT and re-arms the
** engine, which then steps normally.  No counterpart in the reference.
*/
int	anni_optstep_selftest_barrier_timeout(anni_optstep *h, unsigned max_polls, void *stream);

/*
** Diagnostics of the optional one-launch e4m3 form (ANNI_B200_FP8_PIPE=1): polls its blocks have
** spent waiting for each other's tensors since the last call (waits for `stream`, reads and
** clears the counter; -1 on error).  No counterpart in the reference.
*/
long long anni_optstep_pipe_polls(anni_optstep *h, void *stream);

/* Launch geometry in use (blocks of the persistent grid, threads per block). */
int	anni_optstep_grid(anni_optstep *h, int *blocks, int *threads);

/* Number of kernels this library has launched in this process (all entry points). */
uint64_t anni_kernel_launches(void);

#ifdef __cplusplus
}
#endif

#endif
