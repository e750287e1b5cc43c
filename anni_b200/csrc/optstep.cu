/*
** Packed-arena optimizer step for B200 (sm_100a): the kernels and their launchers.
**
** The work is HBM-bound streaming arithmetic, so there are no tensor cores
** here.  What the design spends its effort on instead:
**   - every HBM access of the main path is a coalesced vector load or store with a
**     streaming cache hint: eight elements per thread per chunk in the norm phase, four
**     in the update and quantise phases -- the geometry that keeps the loads queued per
**     SM near the memory system's best point (about 36 KB; more is slower) while leaving
**     enough warps to hide the arithmetic;
**   - the grid is persistent (a multiple of the SM count, all blocks co-resident);
**     chunks are dealt round-robin in super-chunks of four, so the whole grid works
**     inside one contiguous window of every buffer; the norm walks forwards and the
**     update backwards, so that the tail of the gradient shard is still in L2 when it
**     is read the second time;
**   - the global dependency (the gradient norm) is resolved on the device:
**     fixed-order fp64 block partials, a bounded device-wide barrier, and every
**     block derives the same clip factor / skip decision from the same bits;
**   - tensor boundaries, the decay mask and the twin format come from a replicated
**     segment table, looked up once per super-chunk, so one launch covers every tensor.
**
** Arithmetic (what "parity" is measured against): the moments are updated in
** double with the roundings of lang/lm_adam.c:587-591 of the reference
** (products and sum rounded separately, result stored as float), which makes
** m and v bit-identical to the reference's host loop whenever the gradient
** multiplier is bit-identical.  The parameter update runs from the float moments,
** either in float with the SFU's approximate square root and reciprocal (fast mode,
** within an ulp or two of the reference's double expression for ordinary magnitudes)
** or in double with Newton-refined SFU seeds (ANNI_STEP_EXACT_UPDATE, bit-identical
** in all but about one element in 10^5).
*/
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <atomic>
#include "optstep_internal.h"

namespace {

/* ---- small device helpers ------------------------------------------------ */

struct f32x8 {
	float	x[ANNI_VEC];
};

struct f32x4 {
	float	x[ANNI_UVEC];
};

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p)
{
	uint32_t v;

	asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
	return v;
}

/*
** NVSwitch multicast ("multimem") accesses on a multicast address that maps the same buffer of
** every GPU: the load returns the element-wise sum over all copies, reduced inside the switch
** (bf16 pairs accumulated in float); the store lands in every copy.
*/
__device__ __forceinline__ uint4 mc_ld_reduce_bf16x8(const void *mc)
{
	uint4 r;

	asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
	    : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
	return r;
}

__device__ __forceinline__ uint4 mc_ld_reduce_f32x4(const void *mc)
{
	uint4 r;

	asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
	    : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
	return r;
}

__device__ __forceinline__ void mc_st_b64(void *mc, uint2 v)
{
	const unsigned long long x = ((unsigned long long)v.y << 32) | v.x;

	asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" :: "l"(mc), "l"(x) : "memory");
}

__device__ __forceinline__ void mc_st_b32(void *mc, uint32_t v)
{
	asm volatile("multimem.st.relaxed.sys.global.b32 [%0], %1;" :: "l"(mc), "r"(v) : "memory");
}

/*
** The SFU's square root and reciprocal in their single-instruction forms.  These flush
** subnormal inputs and results to zero; the caller keeps its operands out of that range by
** scaling with powers of two (exact), which the forms without .ftz would do with extra
** instructions around the same SFU operation.
*/
__device__ __forceinline__ float sqrt_approx_ftz(float x)
{
	float r;

	asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
	return r;
}

__device__ __forceinline__ float rcp_approx_ftz(float x)
{
	float r;

	asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
	return r;
}

__device__ __forceinline__ f32x8 unpack_bf16x8(uint4 q)
{
	f32x8 r;

	r.x[0] = __uint_as_float(q.x << 16);
	r.x[1] = __uint_as_float(q.x & 0xffff0000u);
	r.x[2] = __uint_as_float(q.y << 16);
	r.x[3] = __uint_as_float(q.y & 0xffff0000u);
	r.x[4] = __uint_as_float(q.z << 16);
	r.x[5] = __uint_as_float(q.z & 0xffff0000u);
	r.x[6] = __uint_as_float(q.w << 16);
	r.x[7] = __uint_as_float(q.w & 0xffff0000u);
	return r;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
	__nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);	/* round to nearest even */

	return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ uint4 pack_bf16x8(const f32x8 &r)
{
	uint4 q;

	q.x = pack_bf16x2(r.x[0], r.x[1]);
	q.y = pack_bf16x2(r.x[2], r.x[3]);
	q.z = pack_bf16x2(r.x[4], r.x[5]);
	q.w = pack_bf16x2(r.x[6], r.x[7]);
	return q;
}

/* eight consecutive elements starting at element index e of a typed buffer */
template <typename T> struct io8;

template <> struct io8<float> {
	static __device__ __forceinline__ f32x8 load(const void *base, uint64_t e)
	{
		const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const float *>(base) + e);
		uint4 a = __ldcs(p);
		uint4 b = __ldcs(p + 1);
		f32x8 r;

		r.x[0] = __uint_as_float(a.x);
		r.x[1] = __uint_as_float(a.y);
		r.x[2] = __uint_as_float(a.z);
		r.x[3] = __uint_as_float(a.w);
		r.x[4] = __uint_as_float(b.x);
		r.x[5] = __uint_as_float(b.y);
		r.x[6] = __uint_as_float(b.z);
		r.x[7] = __uint_as_float(b.w);
		return r;
	}
	/* same, default cache policy: the norm phase wants its last reads to stay in L2 */
	static __device__ __forceinline__ f32x8 load_keep(const void *base, uint64_t e)
	{
		const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const float *>(base) + e);
		uint4 a = p[0];
		uint4 b = p[1];
		f32x8 r;

		r.x[0] = __uint_as_float(a.x);
		r.x[1] = __uint_as_float(a.y);
		r.x[2] = __uint_as_float(a.z);
		r.x[3] = __uint_as_float(a.w);
		r.x[4] = __uint_as_float(b.x);
		r.x[5] = __uint_as_float(b.y);
		r.x[6] = __uint_as_float(b.z);
		r.x[7] = __uint_as_float(b.w);
		return r;
	}
	static __device__ __forceinline__ void store(void *base, uint64_t e, const f32x8 &r)
	{
		uint4 *p = reinterpret_cast<uint4 *>(static_cast<float *>(base) + e);

		__stcs(p, make_uint4(__float_as_uint(r.x[0]), __float_as_uint(r.x[1]),
		    __float_as_uint(r.x[2]), __float_as_uint(r.x[3])));
		__stcs(p + 1, make_uint4(__float_as_uint(r.x[4]), __float_as_uint(r.x[5]),
		    __float_as_uint(r.x[6]), __float_as_uint(r.x[7])));
	}
	static __device__ __forceinline__ void zero(void *base, uint64_t e)
	{
		uint4 *p = reinterpret_cast<uint4 *>(static_cast<float *>(base) + e);

		__stcs(p, make_uint4(0, 0, 0, 0));
		__stcs(p + 1, make_uint4(0, 0, 0, 0));
	}
	static __device__ __forceinline__ float load1(const void *base, uint64_t e)
	{
		return static_cast<const float *>(base)[e];
	}
	static __device__ __forceinline__ void store1(void *base, uint64_t e, float x)
	{
		static_cast<float *>(base)[e] = x;
	}
};

template <> struct io8<__nv_bfloat16> {
	static __device__ __forceinline__ f32x8 load(const void *base, uint64_t e)
	{
		return unpack_bf16x8(__ldcs(reinterpret_cast<const uint4 *>(
		    static_cast<const uint16_t *>(base) + e)));
	}
	static __device__ __forceinline__ f32x8 load_keep(const void *base, uint64_t e)
	{
		return unpack_bf16x8(*reinterpret_cast<const uint4 *>(
		    static_cast<const uint16_t *>(base) + e));
	}
	static __device__ __forceinline__ void store(void *base, uint64_t e, const f32x8 &r)
	{
		__stcs(reinterpret_cast<uint4 *>(static_cast<uint16_t *>(base) + e), pack_bf16x8(r));
	}
	static __device__ __forceinline__ void zero(void *base, uint64_t e)
	{
		__stcs(reinterpret_cast<uint4 *>(static_cast<uint16_t *>(base) + e),
		    make_uint4(0, 0, 0, 0));
	}
	static __device__ __forceinline__ float load1(const void *base, uint64_t e)
	{
		return __uint_as_float((uint32_t)static_cast<const uint16_t *>(base)[e] << 16);
	}
	static __device__ __forceinline__ void store1(void *base, uint64_t e, float x)
	{
		__nv_bfloat16 h = __float2bfloat16_rn(x);

		static_cast<uint16_t *>(base)[e] = *reinterpret_cast<uint16_t *>(&h);
	}
};

/* four consecutive elements starting at element index e: one 16-byte (fp32) or 8-byte (bf16) access */
template <typename T> struct io4;

template <> struct io4<float> {
	static __device__ __forceinline__ f32x4 load(const void *base, uint64_t e)
	{
		const uint4 a = __ldcs(reinterpret_cast<const uint4 *>(static_cast<const float *>(base) + e));
		f32x4 r;

		r.x[0] = __uint_as_float(a.x);
		r.x[1] = __uint_as_float(a.y);
		r.x[2] = __uint_as_float(a.z);
		r.x[3] = __uint_as_float(a.w);
		return r;
	}
	static __device__ __forceinline__ void store(void *base, uint64_t e, const f32x4 &r)
	{
		__stcs(reinterpret_cast<uint4 *>(static_cast<float *>(base) + e),
		    make_uint4(__float_as_uint(r.x[0]), __float_as_uint(r.x[1]), __float_as_uint(r.x[2]),
		    __float_as_uint(r.x[3])));
	}
	/* same, default cache policy: for lines that are read again soon and should wait in L2 */
	static __device__ __forceinline__ void store_keep(void *base, uint64_t e, const f32x4 &r)
	{
		*reinterpret_cast<uint4 *>(static_cast<float *>(base) + e) =
		    make_uint4(__float_as_uint(r.x[0]), __float_as_uint(r.x[1]), __float_as_uint(r.x[2]),
		    __float_as_uint(r.x[3]));
	}
	static __device__ __forceinline__ void zero(void *base, uint64_t e)
	{
		__stcs(reinterpret_cast<uint4 *>(static_cast<float *>(base) + e), make_uint4(0, 0, 0, 0));
	}
};

template <> struct io4<__nv_bfloat16> {
	static __device__ __forceinline__ f32x4 load(const void *base, uint64_t e)
	{
		const uint2 q = __ldcs(reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(base) + e));
		f32x4 r;

		r.x[0] = __uint_as_float(q.x << 16);
		r.x[1] = __uint_as_float(q.x & 0xffff0000u);
		r.x[2] = __uint_as_float(q.y << 16);
		r.x[3] = __uint_as_float(q.y & 0xffff0000u);
		return r;
	}
	static __device__ __forceinline__ void store(void *base, uint64_t e, const f32x4 &r)
	{
		__stcs(reinterpret_cast<uint2 *>(static_cast<uint16_t *>(base) + e),
		    make_uint2(pack_bf16x2(r.x[0], r.x[1]), pack_bf16x2(r.x[2], r.x[3])));
	}
	static __device__ __forceinline__ void zero(void *base, uint64_t e)
	{
		__stcs(reinterpret_cast<uint2 *>(static_cast<uint16_t *>(base) + e), make_uint2(0, 0));
	}
};

/* largest s with seg_off[s] <= x (x inside [seg_off[0], seg_off[n_seg])) */
__device__ __forceinline__ int seg_find(const int64_t *seg_off, int n_seg, int64_t x)
{
	int lo = 0;
	int hi = n_seg - 1;

	while (lo < hi) {
		int mid = (lo + hi + 1) >> 1;

		if (seg_off[mid] <= x)
			lo = mid;
		else
			hi = mid - 1;
	}
	return lo;
}

/*
** Which chunks a block owns.  Chunks are dealt out in "super-chunks" of
** 2^sc_log2 consecutive chunks, round-robin over the grid: iteration `it` of
** block b is chunk ((it >> sc) * grid + b) << sc | (it & mask).  At any moment
** the whole grid then works inside one contiguous window of every buffer
** (good DRAM page locality), while each block still streams runs of
** 2^sc_log2 * ANNI_CHUNK consecutive elements.
*/
struct chunk_walk {
	uint64_t	chunks;	/* chunks in the shard */
	uint64_t	iters;	/* iterations of this block (some of the last may fall outside) */
	uint32_t	sc;
};

/* chunk_log2: log2 of the elements per chunk (ANNI_CHUNK_LOG2 or ANNI_UCHUNK_LOG2) */
__device__ __forceinline__ chunk_walk walk_init(uint64_t n, int sc_log2, int chunk_log2)
{
	chunk_walk w;
	const uint64_t per_round = (uint64_t)gridDim.x << sc_log2;

	w.chunks = (n + ((uint64_t)1 << chunk_log2) - 1) >> chunk_log2;
	w.sc = (uint32_t)sc_log2;
	w.iters = ((w.chunks + per_round - 1) / per_round) << sc_log2;
	return w;
}

/* chunk index of iteration `it`; >= w.chunks means "nothing there" */
__device__ __forceinline__ uint64_t walk_chunk(const chunk_walk &w, uint64_t it)
{
	return ((((it >> w.sc) * gridDim.x + blockIdx.x) << w.sc) | (it & ((1u << w.sc) - 1u)));
}

__device__ __forceinline__ double warp_sum(double v)
{
#pragma unroll
	for (int k = 16; k > 0; k >>= 1)
		v += __shfl_down_sync(0xffffffffu, v, k);
	return v;
}

/* Block sum in a fixed order; the result is valid in thread 0. */
__device__ __forceinline__ double block_sum(double v)
{
	__shared__ double s_w[ANNI_THREADS / 32];
	const int lane = threadIdx.x & 31;
	const int w = threadIdx.x >> 5;

	v = warp_sum(v);
	if (lane == 0)
		s_w[w] = v;
	__syncthreads();
	if (threadIdx.x == 0) {
		v = 0.0;
#pragma unroll
		for (int k = 0; k < ANNI_THREADS / 32; k++)
			v += s_w[k];
	}
	return v;
}

/*
** Device-wide barrier with a bounded wait.  All blocks of the grid are
** co-resident (cooperative launch), so the wait ends as soon as the slowest
** block arrives; the poll limit only matters if something is badly wrong, in
** which case the block records the error and the kernel returns without
** touching the parameters.  Returns false on timeout (uniform over the block).
*/
__device__ __forceinline__ bool grid_barrier(anni_control *ctl, uint32_t target,
	uint32_t max_polls = ANNI_WAIT_POLLS)
{
	__shared__ int s_ok;

	__syncthreads();
	if (threadIdx.x == 0) {
		uint32_t polls = 0;
		int ok = 1;

		__threadfence();
		atomicAdd(&ctl->bar_count, 1u);
		while (ld_acquire_u32(&ctl->bar_count) < target) {
			__nanosleep(32);
			if (++polls > max_polls) {
				ok = 0;
				atomicExch(&ctl->error, ANNI_E_BARRIER_TIMEOUT);
				break;
			}
		}
		__threadfence();
		s_ok = ok;
	}
	__syncthreads();
	return s_ok != 0;
}

/* Sum of the block partials in index order; every thread of the block gets it. */
__device__ __forceinline__ double sum_partials(const anni_control *ctl, int nparts)
{
	__shared__ double s_total;

	if (threadIdx.x < 32) {
		const volatile double *p = ctl->partials;
		double v = 0.0;

		for (int k = threadIdx.x; k < nparts; k += 32)
			v += p[k];
		v = warp_sum(v);
		if (threadIdx.x == 0)
			s_total = v;
	}
	__syncthreads();
	return s_total;
}

/* ---- phase A: sum of squares of this block's chunks ---------------------- */

template <typename GradT>
__device__ __forceinline__ void norm_accumulate(const f32x8 &g, double &acc0, double &acc1)
{
	/* squares and their sum in double: the skip decision and the clip factor then
	** agree with a double accumulation to the last bits */
#pragma unroll
	for (int k = 0; k < ANNI_VEC; k += 2) {
		const double g0 = (double)g.x[k];
		const double g1 = (double)g.x[k + 1];

		acc0 = fma(g0, g0, acc0);
		acc1 = fma(g1, g1, acc1);
	}
}

template <typename GradT>
__device__ __forceinline__ double norm_phase(const anni_launch &a)
{
	const chunk_walk w = walk_init(a.n, a.sc_log2, ANNI_CHUNK_LOG2);
	double acc0 = 0.0;
	double acc1 = 0.0;
	const uint64_t t8 = (uint64_t)threadIdx.x * ANNI_VEC;
	uint64_t it = 0;

	/* four chunks per trip while whole aligned chunks last: four independent 16-byte loads in flight */
	if (a.aligned) {
		for (; it + 4 <= w.iters; it += 4) {
			const uint64_t c0 = walk_chunk(w, it);
			const uint64_t c1 = walk_chunk(w, it + 1);
			const uint64_t c2 = walk_chunk(w, it + 2);
			const uint64_t c3 = walk_chunk(w, it + 3);
			const uint64_t cmax = max(max(c0, c1), max(c2, c3));

			if ((cmax + 1) * ANNI_CHUNK > a.n)
				break;
			const f32x8 g0 = io8<GradT>::load_keep(a.grad, c0 * ANNI_CHUNK + t8);
			const f32x8 g1 = io8<GradT>::load_keep(a.grad, c1 * ANNI_CHUNK + t8);
			const f32x8 g2 = io8<GradT>::load_keep(a.grad, c2 * ANNI_CHUNK + t8);
			const f32x8 g3 = io8<GradT>::load_keep(a.grad, c3 * ANNI_CHUNK + t8);

			norm_accumulate<GradT>(g0, acc0, acc1);
			norm_accumulate<GradT>(g1, acc0, acc1);
			norm_accumulate<GradT>(g2, acc0, acc1);
			norm_accumulate<GradT>(g3, acc0, acc1);
		}
	}
	for (; it < w.iters; it++) {
		const uint64_t c = walk_chunk(w, it);
		const uint64_t e = c * ANNI_CHUNK + t8;

		if (c >= w.chunks)
			continue;
		if (a.aligned && e + ANNI_VEC <= a.n) {
			const f32x8 g = io8<GradT>::load_keep(a.grad, e);

			norm_accumulate<GradT>(g, acc0, acc1);
		} else {
			for (int k = 0; k < ANNI_VEC; k++)
				if (e + k < a.n) {
					double g = (double)io8<GradT>::load1(a.grad, e + k);

					acc0 = fma(g, g, acc0);
				}
		}
	}
	return acc0 + acc1;
}

/* ---- the decision every block takes from the same bits --------------------- */

struct decision {
	double	coef;	/* multiplier of the raw gradient */
	double	norm;
	bool	skip;
};

__device__ __forceinline__ decision decide(const anni_launch &a, double ss, double nonfinite,
	double loss_scale)
{
	decision d;
	double gs = a.grad_scale;

	if ((a.flags & ANNI_STEP_DEV_LOSS_SCALE) && loss_scale > 0.0)
		gs = gs / loss_scale;
	d.coef = gs;
	d.norm = 0.0;
	d.skip = false;
	if (a.flags & ANNI_LAUNCH_NEED_NORM) {
		d.norm = sqrt(ss) * fabs(gs);
		if ((a.flags & ANNI_STEP_CHECK_FINITE) && (!isfinite(d.norm) || nonfinite > 0.0))
			d.skip = true;
		else if (a.clip > 0.0 && d.norm > a.clip)
			d.coef = gs * (a.clip / (d.norm + 1e-12));
	}
	return d;
}

/* ---- phase B: AdamW on one element ----------------------------------------- */

template <bool EXACT>
__device__ __forceinline__ void adam_elem(const anni_launch &a, double coef, float lrwd,
	float gf, float &p, float &m, float &v)
{
	/* moments: the reference's double expression, each product and the sum rounded on its own */
	const double g = __dmul_rn((double)gf, coef);
	const double md = __dadd_rn(__dmul_rn(a.b1, (double)m), __dmul_rn(a.omb1, g));
	const double vd = __dadd_rn(__dmul_rn(a.b2, (double)v), __dmul_rn(__dmul_rn(a.omb2, g), g));

	m = __double2float_rn(md);
	v = __double2float_rn(vd);
	/*
	** p -= lr * (m/bc1) / (sqrt(v/bc2) + eps), then p -= lr*wd*p on the stored
	** value.  The quotient uses the SFU square root and reciprocal (about one
	** ulp each): the update term carries a relative error of a few 1e-7, which
	** moves p by far less than one ulp unless p itself is of the size of the
	** update.  Every product is rounded on its own (no contraction).
	*/
	if (EXACT) {
		/*
		** The reference's double expression lr*(m/bc1)/(sqrt(v/bc2)+eps) from the
		** rounded float moments: reciprocal square root and reciprocal start from
		** the SFU's 64-bit seeds (about 20 bits) and take one Newton step each
		** (relative error ~1e-12), so p - u rounds to the reference's float in
		** all but about one element in ten million.
		*/
		const double vr = (double)v;
		const double x = vr * a.ibc2d;
		const double hx = vr * (0.5 * a.ibc2d);
		double y;
		double q;

		asm("rsqrt.approx.ftz.f64 %0, %1;" : "=d"(y) : "d"(x));
		y = y * fma(-hx * y, y, 1.5);
		const double dn = (v > 0.0f ? x * y : 0.0) + a.epsd;

		asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(q) : "d"(dn));
		q = fma(fma(-dn, q, 1.0), q, q);
		const float p1 = __double2float_rn((double)p - (a.lrbc1d * (double)m) * q);

		/* decay on the stored float, in double as the reference does, rounded once */
		p = lrwd != 0.0f ? __double2float_rn(fma(-a.lrwdd, (double)p1, (double)p1)) : p1;
		return;
	}
	/*
	** den = sqrt(v / bc2) + eps and upd = (lr / bc1 * m) / den, carried at other binary
	** scales: s = sqrt(2^24 v / bc2) = 2^12 sqrt(v / bc2), so no subnormal v is flushed;
	** den40 = 2^28 s + 2^40 eps = 2^40 den in one fused step (the same single rounding as
	** the plain sum), never subnormal unless it is zero; the factor 2^40 returns through lr.
	*/
	const float s = sqrt_approx_ftz(__fmul_rn(v, a.ibc2_s24));
	const float den40 = __fmaf_rn(s, 268435456.0f, a.eps_s40);
	const float upd = __fmul_rn(__fmul_rn(a.lrbc1_s40, m), rcp_approx_ftz(den40));

	p = __fsub_rn(p, upd);
	p = __fmaf_rn(-lrwd, p, p);
}

/*
** How a kernel variant treats what follows the plain update: MODE_PLAIN clears the bound
** gradient buffer; MODE_PIPE (one-launch step only) also quantises e4m3 twins behind the
** update; MODE_ARENA (update kernel only) clears every part of the rank's full gradient arena
** instead of the bound buffer.  Compile-time, so that the plain variants carry none of the
** other two's registers.
*/
enum { MODE_PLAIN = 0, MODE_PIPE = 1, MODE_ARENA = 2 };

/* "the step leaves the gradients zeroed": the bound buffer, or every part of the rank's full arena */
template <typename GradT, int MODE>
__device__ __forceinline__ void zero_grad4(const anni_launch &a, uint64_t e)
{
	if (MODE == MODE_ARENA) {
		for (int k = 0; k < a.zero_parts; k++)
			if (k + 1 != a.zero_done)
				io4<GradT>::zero(a.zero_base, (uint64_t)k * a.zero_stride + e);
	} else
		io4<GradT>::zero(a.grad, e);
}

template <typename GradT, int MODE>
__device__ __forceinline__ void zero_grad1(const anni_launch &a, uint64_t i)
{
	if (MODE == MODE_ARENA) {
		for (int k = 0; k < a.zero_parts; k++)
			if (k + 1 != a.zero_done)
				io8<GradT>::store1(a.zero_base, (uint64_t)k * a.zero_stride + i, 0.0f);
	} else
		io8<GradT>::store1(a.grad, i, 0.0f);
}

template <typename GradT, typename StateT, bool EXACT, int MODE>
__device__ __forceinline__ void update_chunk_vec(const anni_launch &a, uint64_t e, double coef,
	uint32_t sflags, float &tmax, uint64_t seg_base, int64_t pack_off, uint32_t pack_ld,
	uint32_t pack_cols)
{
	const float lrwd = (sflags & ANNI_SEG_WD) ? a.lrwd : 0.0f;
	f32x4 g = io4<GradT>::load(a.grad, e);
	f32x4 p = io4<float>::load(a.master, e);
	f32x4 m = io4<StateT>::load(a.m, e);
	f32x4 v = io4<StateT>::load(a.v, e);

#pragma unroll
	for (int k = 0; k < ANNI_UVEC; k++)
		adam_elem<EXACT>(a, coef, lrwd, g.x[k], p.x[k], m.x[k], v.x[k]);
	if (MODE == MODE_PIPE && (sflags & ANNI_SEG_TWIN_FP8) && !(a.flags & ANNI_LAUNCH_PIPE_STREAM))
		io4<float>::store_keep(a.master, e, p);	/* read back for its e4m3 code while still in L2 */
	else
		io4<float>::store(a.master, e, p);
	io4<StateT>::store(a.m, e, m);
	io4<StateT>::store(a.v, e, v);
	if ((sflags & ANNI_SEG_TWIN_BF16) && a.twin16) {
		if (a.mc_twin) {
			/* the all-gather, fused: ONE multicast store, replicated by the switch into every rank's arena */
			mc_st_b64(a.mc_twin + e, make_uint2(pack_bf16x2(p.x[0], p.x[1]), pack_bf16x2(p.x[2], p.x[3])));
		} else if (a.n_peers > 0) {
			/* without multicast: this shard's twins stored into every rank's arena one by one */
			for (int k = 0; k < a.n_peers; k++)
				io4<__nv_bfloat16>::store(a.twin_peer[k], e, p);
		} else
			io4<__nv_bfloat16>::store(a.twin16, e, p);
	}
	if (sflags & ANNI_SEG_TWIN_FP8) {
#pragma unroll
		for (int k = 0; k < ANNI_UVEC; k++)
			tmax = fmaxf(tmax, fabsf(p.x[k]));
	}
	if (pack_ld != 0) {
		/* the same twin once more, as a block of the layer's packed [Wq|Wk|Wv] matrix;
		** four consecutive elements stay inside one row because cols % 4 == 0 (checked on the host) */
		const uint32_t ws = (uint32_t)(e - seg_base);
		const uint32_t r = ws / pack_cols;

		io4<__nv_bfloat16>::store(a.qkv_packed, (uint64_t)pack_off + (uint64_t)r * pack_ld
		    + (ws - r * pack_cols), p);
	}
	if (a.flags & ANNI_STEP_ZERO_GRAD)
		zero_grad4<GradT, MODE>(a, e);
}

/* element-wise path for chunks that cross a tensor boundary, the arena end, or unaligned buffers */
template <typename GradT, typename StateT, bool EXACT, int MODE>
__device__ __forceinline__ void update_chunk_scalar(const anni_launch &a, uint64_t e, double coef,
	bool skip)
{
	for (int k = 0; k < ANNI_UVEC; k++) {
		const uint64_t i = e + k;

		if (i >= a.n)
			break;
		if (!skip) {
			const int s = seg_find(a.seg_off, a.n_seg, (int64_t)(a.arena_off + i));
			const uint32_t sflags = a.seg_flags[s];
			const float lrwd = (sflags & ANNI_SEG_WD) ? a.lrwd : 0.0f;
			float p = a.master[i];
			float m = io8<StateT>::load1(a.m, i);
			float v = io8<StateT>::load1(a.v, i);

			adam_elem<EXACT>(a, coef, lrwd, io8<GradT>::load1(a.grad, i), p, m, v);
			a.master[i] = p;
			io8<StateT>::store1(a.m, i, m);
			io8<StateT>::store1(a.v, i, v);
			if ((sflags & ANNI_SEG_TWIN_BF16) && a.twin16) {
				if (a.n_peers > 0) {
					for (int q = 0; q < a.n_peers; q++)
						io8<__nv_bfloat16>::store1(a.twin_peer[q], i, p);
				} else
					io8<__nv_bfloat16>::store1(a.twin16, i, p);
			}
			if (sflags & ANNI_SEG_TWIN_FP8)
				atomicMax(reinterpret_cast<int *>(&a.seg_amax[s]),
				    __float_as_int(fabsf(p)));
			if (a.seg_aux && a.seg_aux[s].pack_ld != 0) {
				const anni_seg_derived ax = a.seg_aux[s];
				const uint32_t ws = (uint32_t)((int64_t)(a.arena_off + i) - a.seg_off[s]);
				const uint32_t r = ws / (uint32_t)ax.cols;

				io8<__nv_bfloat16>::store1(a.qkv_packed, (uint64_t)ax.pack_off
				    + (uint64_t)r * (uint32_t)ax.pack_ld + (ws - r * (uint32_t)ax.cols), p);
			}
		}
		if (a.flags & ANNI_STEP_ZERO_GRAD)
			zero_grad1<GradT, MODE>(a, i);
	}
}

__device__ __forceinline__ void amax_flush(const anni_launch &a, int seg, float &tmax)
{
	float w = tmax;

#pragma unroll
	for (int k = 16; k > 0; k >>= 1)
		w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, k));
	if ((threadIdx.x & 31) == 0 && w > 0.0f)
		atomicMax(reinterpret_cast<int *>(&a.seg_amax[seg]), __float_as_int(w));
	tmax = 0.0f;
}

/* one chunk the general way: tensor looked up from scratch, element-wise when the chunk is not whole */
template <typename GradT, typename StateT, bool EXACT, int MODE>
__device__ __forceinline__ void update_chunk_general(const anni_launch &a, const decision &d, uint64_t base,
	uint64_t t4, float &tmax, int &amax_seg)
{
	const int64_t abase = (int64_t)(a.arena_off + base);
	const int seg = seg_find(a.seg_off, a.n_seg, abase);
	const bool whole = a.aligned && base + ANNI_UCHUNK <= a.n
	    && abase + ANNI_UCHUNK <= a.seg_off[seg + 1];

	if (whole && !d.skip) {
		const uint32_t sflags = a.seg_flags[seg];

		if (amax_seg != seg) {
			if (amax_seg >= 0)
				amax_flush(a, amax_seg, tmax);
			amax_seg = (sflags & ANNI_SEG_TWIN_FP8) ? seg : -1;
		}
		if (a.seg_aux) {
			const anni_seg_derived ax = a.seg_aux[seg];

			update_chunk_vec<GradT, StateT, EXACT, MODE>(a, base + t4, d.coef, sflags, tmax,
			    (uint64_t)a.seg_off[seg] - a.arena_off, ax.pack_off, (uint32_t)ax.pack_ld,
			    (uint32_t)ax.cols);
		} else
			update_chunk_vec<GradT, StateT, EXACT, MODE>(a, base + t4, d.coef, sflags, tmax, 0, 0, 0, 1);
	} else if (whole) {
		zero_grad4<GradT, MODE>(a, base + t4);	/* skipped step: only the gradients change */
	} else
		update_chunk_scalar<GradT, StateT, EXACT, MODE>(a, base + t4, d.coef, d.skip);
}

/* dequantisation scale of a tensor from its amax (num/gpu_cuda.cu:927-938 of the reference) */
__device__ __forceinline__ float fp8_scale(float amax)
{
	float s = amax;

	if (!(s > 0.0f) || !isfinite(s))
		s = 1e-8f;
	s = __fdiv_rn(s, 448.0f);
	return s < 1e-12f ? 1e-12f : s;
}

/* e4m3 codes of four masters (already multiplied by 1/scale on the way in), packed little-endian */
__device__ __forceinline__ uint32_t e4m3x4(const f32x4 &p, float inv)
{
	return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(p.x[0] * inv, p.x[1] * inv), __NV_SATFINITE, __NV_E4M3)
	    | ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(p.x[2] * inv, p.x[3] * inv), __NV_SATFINITE,
	    __NV_E4M3) << 16);
}

__device__ __forceinline__ void store_e4m3x4(const anni_launch &a, uint64_t e, uint32_t q)
{
	if (a.mc_twin8)
		mc_st_b32(a.mc_twin8 + e, q);
	else if (a.n_peers > 0) {
		for (int k = 0; k < a.n_peers; k++)
			__stcs(reinterpret_cast<uint32_t *>(a.twin8_peer[k] + e), q);
	} else
		__stcs(reinterpret_cast<uint32_t *>(a.twin8 + e), q);
}

/*
** One-launch step with e4m3 twins: the quantiser runs BEHIND the update, tensor by tensor,
** instead of as a second pass over the whole arena after a grid barrier.  A tensor's codes
** need its amax, i.e. every block must have finished updating it; re-reading its fresh
** master from HBM afterwards costs 4 bytes per element.  So each block reports a tensor as
** soon as its own (descending) walk has left it behind -- after flushing its amax share --
** and from then on slips a little of that tensor's quantising in after every super-chunk it
** updates: one trip of four chunks per round, two while it has a backlog.  The quantiser's
** loads hit the 126 MB L2 (the masters of such tensors are stored with the default policy,
** everything else streams through with evict-first hints; measured: 91 % of them), and because
** they are spread over the update's rounds they overlap its HBM traffic instead of replacing
** it.  (Measured, it still does not pay: the step is 3-6 % slower than with a quantise phase of
** its own after a second grid barrier, so this form is opt-in.)  Nobody waits inside the walk: a tensor that the rest of the grid has not left yet is
** simply tried again next round.  Only after its last super-chunk does a block wait for the
** tensors still open, with the same bound as the grid barrier, giving up at once when any
** block has raised an error.
*/
__device__ __forceinline__ bool pipe_wants(const anni_launch &a, int s)
{
	return (a.seg_flags[s] & ANNI_SEG_TWIN_FP8) && !(a.seg_aux && a.seg_aux[s].fp8_t_off >= 0);
}

/* this block will not touch tensor s again (block-uniform call) */
__device__ __forceinline__ void pipe_report(const anni_launch &a, int s)
{
	if (!pipe_wants(a, s))
		return;
	__syncthreads();
	if (threadIdx.x == 0) {
		__threadfence();
		atomicAdd(&a.seg_done[s], 1u);
	}
}

/* the tensor a block is quantising its share of (all fields block-uniform) */
struct pipe_state {
	uint64_t	c;	/* this block's next chunk of the tensor */
	uint64_t	c_hi;	/* one past the tensor's last chunk */
	uint64_t	lo;	/* the tensor inside the shard: elements [lo, hi) */
	uint64_t	hi;
	float		inv;	/* 1 / scale, once the tensor is complete */
	int		s;	/* tensor, or -1: none open */
	bool		ready;	/* every block has reported it; inv is valid */
};

/* opens tensor s; false when there is nothing to quantise in it for anybody in this shard */
__device__ __forceinline__ bool pipe_open(const anni_launch &a, int s, pipe_state &q)
{
	if (!pipe_wants(a, s))
		return false;
	const int64_t t_lo = max(a.seg_off[s], (int64_t)a.arena_off) - (int64_t)a.arena_off;
	const int64_t t_hi = min(a.seg_off[s + 1], (int64_t)(a.arena_off + a.n)) - (int64_t)a.arena_off;

	if (t_lo >= t_hi)
		return false;
	q.s = s;
	q.ready = false;
	q.lo = (uint64_t)t_lo;
	q.hi = (uint64_t)t_hi;
	q.c = (q.lo >> ANNI_UCHUNK_LOG2) + blockIdx.x;
	q.c_hi = (q.hi + ANNI_UCHUNK - 1) >> ANNI_UCHUNK_LOG2;
	return true;
}

/*
** Has the whole grid reported the open tensor?  1: yes (q.inv set), 0: not yet (only when
** `wait` is false), -1: the bounded wait gave up.  Block-uniform; one block-wide
** synchronisation per call.
*/
__device__ __forceinline__ int pipe_poll(const anni_launch &a, pipe_state &q, bool wait)
{
	__shared__ int s_state;

	__syncthreads();
	if (threadIdx.x == 0) {
		uint32_t polls = 0;
		int state = 1;

		while (ld_acquire_u32(&a.seg_done[q.s]) < gridDim.x) {
			if (!wait) {
				state = 0;
				break;
			}
			__nanosleep(32);
			if (++polls > ANNI_WAIT_POLLS
			    || ld_acquire_u32(reinterpret_cast<const uint32_t *>(&a.ctl->error)) != 0) {
				state = -1;
				atomicCAS(&a.ctl->error, 0, ANNI_E_BARRIER_TIMEOUT);
				break;
			}
		}
		if (polls)
			atomicAdd(&a.ctl->pipe_polls, polls);
		__threadfence();
		s_state = state;
	}
	__syncthreads();
	const int state = s_state;

	if (state == 1) {
		const float scale = fp8_scale(__ldcg(&a.seg_amax[q.s]));

		q.inv = __fdiv_rn(1.0f, scale);
		q.ready = true;
		if (blockIdx.x == 0 && threadIdx.x == 0)
			a.seg_scale[q.s] = scale;
	}
	return state;
}

/* one trip: up to four of this block's chunks of the open tensor; true when the tensor is finished */
__device__ __forceinline__ bool pipe_trip(const anni_launch &a, pipe_state &q)
{
	const uint64_t t4 = (uint64_t)threadIdx.x * ANNI_UVEC;
	const uint64_t G = gridDim.x;
	const uint64_t c = q.c;

	if (c >= q.c_hi)
		return true;
	q.c = c + 4 * G;
	/* four whole chunks: their loads issued together */
	if (a.aligned && (c << ANNI_UCHUNK_LOG2) >= q.lo && ((c + 3 * G + 1) << ANNI_UCHUNK_LOG2) <= q.hi) {
		const uint64_t e0 = (c << ANNI_UCHUNK_LOG2) + t4;
		const uint64_t st = G << ANNI_UCHUNK_LOG2;
		const f32x4 p0 = io4<float>::load(a.master, e0);
		const f32x4 p1 = io4<float>::load(a.master, e0 + st);
		const f32x4 p2 = io4<float>::load(a.master, e0 + 2 * st);
		const f32x4 p3 = io4<float>::load(a.master, e0 + 3 * st);

		store_e4m3x4(a, e0, e4m3x4(p0, q.inv));
		store_e4m3x4(a, e0 + st, e4m3x4(p1, q.inv));
		store_e4m3x4(a, e0 + 2 * st, e4m3x4(p2, q.inv));
		store_e4m3x4(a, e0 + 3 * st, e4m3x4(p3, q.inv));
		return q.c >= q.c_hi;
	}
	for (int k = 0; k < 4; k++) {
		const uint64_t ck = c + (uint64_t)k * G;
		const uint64_t e = (ck << ANNI_UCHUNK_LOG2) + t4;

		if (ck >= q.c_hi)
			break;
		if (a.aligned && (ck << ANNI_UCHUNK_LOG2) >= q.lo && ((ck + 1) << ANNI_UCHUNK_LOG2) <= q.hi) {
			store_e4m3x4(a, e, e4m3x4(io4<float>::load(a.master, e), q.inv));
			continue;
		}
		for (int j = 0; j < ANNI_UVEC; j++)	/* the tensor's ragged ends, its own elements only */
			if (e + j >= q.lo && e + j < q.hi)
				a.twin8[e + j] = (uint8_t)__nv_cvt_float_to_fp8(a.master[e + j] * q.inv,
				    __NV_SATFINITE, __NV_E4M3);
	}
	return q.c >= q.c_hi;
}

/*
** Up to `trips` trips on the tensors this block has reported down to (not including) rep_hi,
** highest first.  wait = false: a tensor the grid has not finished is left for the next call.
** False when a bounded wait gave up.
*/
__device__ __forceinline__ bool pipe_work(const anni_launch &a, pipe_state &q, int &q_hi, int rep_hi,
	int trips, bool wait)
{
	while (trips > 0) {
		if (q.s < 0) {
			if (q_hi <= rep_hi)
				return true;		/* nothing reported that is still to do */
			if (!pipe_open(a, q_hi--, q))
				continue;
		}
		if (!q.ready) {
			const int state = pipe_poll(a, q, wait);

			if (state < 0)
				return false;
			if (state == 0)
				return true;		/* not complete yet: next round */
		}
		if (pipe_trip(a, q))
			q.s = -1;
		trips--;
	}
	return true;
}

/*
** The blocks walk their super-chunks (2^sc_log2 consecutive chunks) from the last to the
** first.  A super-chunk that lies wholly inside the shard and inside one tensor -- all but a
** few hundred of them -- takes the short road: tensor flags looked up once, then nothing
** but loads, arithmetic and stores per chunk.  The others go chunk by chunk the general way.
*/
template <typename GradT, typename StateT, bool EXACT, int MODE>
__device__ __forceinline__ bool update_phase(const anni_launch &a, const decision &d)
{
	const chunk_walk w = walk_init(a.n, a.sc_log2, ANNI_UCHUNK_LOG2);
	const uint64_t t4 = (uint64_t)threadIdx.x * ANNI_UVEC;
	const uint32_t per = 1u << w.sc;			/* chunks per super-chunk */
	const uint64_t span = (uint64_t)ANNI_UCHUNK << w.sc;	/* elements per super-chunk */
	float tmax = 0.0f;
	int seg = -1;
	int amax_seg = -1;
	int rep_hi = a.n_seg - 1;	/* PIPE: highest tensor this block has not reported yet */
	int q_hi = a.n_seg - 1;		/* PIPE: highest tensor this block has not opened for quantising yet */
	pipe_state q;

	q.s = -1;
	q.ready = false;
	q.c = q.c_hi = q.lo = q.hi = 0;
	q.inv = 0.0f;

	if (d.skip && !(a.flags & ANNI_STEP_ZERO_GRAD))
		return true;
	/* backwards: the chunks read last by the norm phase are the likeliest to sit in L2 */
	for (uint64_t r = w.iters >> w.sc; r > 0; r--) {
		const uint64_t c0 = ((r - 1) * gridDim.x + blockIdx.x) << w.sc;
		const uint64_t base0 = c0 * ANNI_UCHUNK;
		const int64_t alo = (int64_t)(a.arena_off + base0);

		if (c0 >= w.chunks)
			continue;
		if (MODE == MODE_PIPE && !d.skip) {
			const int64_t top = alo + (int64_t)span;	/* this and all later super-chunks lie below */

			while (rep_hi >= 0 && a.seg_off[rep_hi] >= top) {
				if (amax_seg >= rep_hi) {
					amax_flush(a, amax_seg, tmax);
					amax_seg = -1;
				}
				pipe_report(a, rep_hi--);
			}
			/* a little quantising per round; more while further tensors are waiting behind the open one */
			if ((q.s >= 0 || q_hi > rep_hi)
			    && !pipe_work(a, q, q_hi, rep_hi, q_hi - rep_hi >= 2 ? a.pipe_lag : 1, false))
				return false;
		}
		if (seg < 0)
			seg = seg_find(a.seg_off, a.n_seg, alo);
		while (alo < a.seg_off[seg])
			seg--;
		if (!d.skip && a.aligned && base0 + span <= a.n && alo + (int64_t)span <= a.seg_off[seg + 1]) {
			const uint32_t sflags = a.seg_flags[seg];

			if (amax_seg != seg) {
				if (amax_seg >= 0)
					amax_flush(a, amax_seg, tmax);
				amax_seg = (sflags & ANNI_SEG_TWIN_FP8) ? seg : -1;
			}
			if (a.seg_aux) {
				const anni_seg_derived ax = a.seg_aux[seg];
				const uint64_t seg_base = (uint64_t)a.seg_off[seg] - a.arena_off;

#pragma unroll 1
				for (uint32_t k = per; k > 0; k--)
					update_chunk_vec<GradT, StateT, EXACT, MODE>(a, base0 + (uint64_t)(k - 1) * ANNI_UCHUNK + t4,
					    d.coef, sflags, tmax, seg_base, ax.pack_off, (uint32_t)ax.pack_ld,
					    (uint32_t)ax.cols);
			} else {
#pragma unroll 1
				for (uint32_t k = per; k > 0; k--)
					update_chunk_vec<GradT, StateT, EXACT, MODE>(a, base0 + (uint64_t)(k - 1) * ANNI_UCHUNK + t4,
					    d.coef, sflags, tmax, 0, 0, 0, 1);
			}
		} else {
			for (uint32_t k = per; k > 0; k--)
				if (c0 + (k - 1) < w.chunks)
					update_chunk_general<GradT, StateT, EXACT, MODE>(a, d, base0 + (uint64_t)(k - 1) * ANNI_UCHUNK,
					    t4, tmax, amax_seg);
		}
	}
	if (amax_seg >= 0)
		amax_flush(a, amax_seg, tmax);
	if (MODE == MODE_PIPE && !d.skip) {
		/* the walk is over: report what is left, then quantise what is left */
		while (rep_hi >= 0)
			pipe_report(a, rep_hi--);
		while (q.s >= 0 || q_hi >= 0)
			if (!pipe_work(a, q, q_hi, -1, 1 << 20, true))
				return false;
	}
	return true;
}

/* ---- phase C: e4m3 twins of the fresh master ------------------------------- */

/* one chunk the general way: element-wise when it is not whole */
__device__ __forceinline__ void quantize_chunk_general(const anni_launch &a, uint64_t base, uint64_t t4)
{
	const int64_t abase = (int64_t)(a.arena_off + base);
	const int seg = seg_find(a.seg_off, a.n_seg, abase);

	if (a.aligned && base + ANNI_UCHUNK <= a.n && abase + ANNI_UCHUNK <= a.seg_off[seg + 1]) {
		if ((a.seg_flags[seg] & ANNI_SEG_TWIN_FP8) && !(a.seg_aux && a.seg_aux[seg].fp8_t_off >= 0)) {
			const float inv = __fdiv_rn(1.0f, fp8_scale(a.seg_amax[seg]));

			store_e4m3x4(a, base + t4, e4m3x4(io4<float>::load(a.master, base + t4), inv));
		}
		return;
	}
	for (int k = 0; k < ANNI_UVEC; k++) {
		const uint64_t i = base + t4 + k;

		if (i >= a.n)
			break;
		const int s = seg_find(a.seg_off, a.n_seg, (int64_t)(a.arena_off + i));

		if ((a.seg_flags[s] & ANNI_SEG_TWIN_FP8) && !(a.seg_aux && a.seg_aux[s].fp8_t_off >= 0)) {
			const float inv = __fdiv_rn(1.0f, fp8_scale(a.seg_amax[s]));
			const uint8_t q8 = (uint8_t)__nv_cvt_float_to_fp8(a.master[i] * inv,
			    __NV_SATFINITE, __NV_E4M3);

			if (a.n_peers > 0) {
				for (int q = 0; q < a.n_peers; q++)
					a.twin8_peer[q][i] = q8;
			} else
				a.twin8[i] = q8;
		}
	}
}

/*
** Super-chunk by super-chunk, as the update phase: a super-chunk of four chunks inside one
** tensor has its scale looked up once and its four 128-bit loads per thread issued together
** (a single load in flight per thread leaves the memory system half idle: 3.4 TB/s).
*/
__device__ __forceinline__ void quantize_phase(const anni_launch &a)
{
	const chunk_walk w = walk_init(a.n, a.sc_log2, ANNI_UCHUNK_LOG2);
	const uint64_t t4 = (uint64_t)threadIdx.x * ANNI_UVEC;
	const uint32_t per = 1u << w.sc;
	const uint64_t span = (uint64_t)ANNI_UCHUNK << w.sc;
	int seg = -1;

	if (!a.twin8)
		return;
	if (blockIdx.x == 0)
		for (int s = threadIdx.x; s < a.n_seg; s += blockDim.x)
			if (a.seg_flags[s] & ANNI_SEG_TWIN_FP8)
				a.seg_scale[s] = fp8_scale(a.seg_amax[s]);
	for (uint64_t r = 0; r < (w.iters >> w.sc); r++) {
		const uint64_t c0 = (r * gridDim.x + blockIdx.x) << w.sc;
		const uint64_t base0 = c0 * ANNI_UCHUNK;
		const int64_t alo = (int64_t)(a.arena_off + base0);

		if (c0 >= w.chunks)
			continue;
		if (seg < 0)
			seg = seg_find(a.seg_off, a.n_seg, alo);
		while (alo >= a.seg_off[seg + 1])
			seg++;
		if (w.sc == 2 && a.aligned && base0 + span <= a.n && alo + (int64_t)span <= a.seg_off[seg + 1]) {
			if ((a.seg_flags[seg] & ANNI_SEG_TWIN_FP8) && !(a.seg_aux && a.seg_aux[seg].fp8_t_off >= 0)) {
				const float inv = __fdiv_rn(1.0f, fp8_scale(a.seg_amax[seg]));
				const uint64_t e0 = base0 + t4;
				const f32x4 p0 = io4<float>::load(a.master, e0);
				const f32x4 p1 = io4<float>::load(a.master, e0 + ANNI_UCHUNK);
				const f32x4 p2 = io4<float>::load(a.master, e0 + 2 * ANNI_UCHUNK);
				const f32x4 p3 = io4<float>::load(a.master, e0 + 3 * ANNI_UCHUNK);

				store_e4m3x4(a, e0, e4m3x4(p0, inv));
				store_e4m3x4(a, e0 + ANNI_UCHUNK, e4m3x4(p1, inv));
				store_e4m3x4(a, e0 + 2 * ANNI_UCHUNK, e4m3x4(p2, inv));
				store_e4m3x4(a, e0 + 3 * ANNI_UCHUNK, e4m3x4(p3, inv));
			}
		} else {
			for (uint32_t k = 0; k < per; k++)
				if (c0 + k < w.chunks)
					quantize_chunk_general(a, base0 + (uint64_t)k * ANNI_UCHUNK, t4);
		}
	}
}

/* ---- epilogue: the last block to finish closes the step --------------------- */

__device__ __forceinline__ void step_epilogue(anni_control *ctl, bool skipped)
{
	__syncthreads();
	if (threadIdx.x != 0)
		return;
	__threadfence();
	if (atomicAdd(&ctl->done_ticket, 1u) != gridDim.x - 1)
		return;
	/* every block has read the loss scale and passed every barrier by now */
	if (ctl->loss_scale > 0.0) {
		if (skipped) {
			double s = ctl->loss_scale * ctl->ls_backoff;

			ctl->loss_scale = s < ctl->ls_min ? ctl->ls_min : s;
			ctl->good_steps = 0;
		} else if (++ctl->good_steps >= ctl->ls_interval && ctl->ls_interval > 0) {
			double s = ctl->loss_scale * ctl->ls_growth;

			ctl->loss_scale = s > ctl->ls_max ? ctl->ls_max : s;
			ctl->good_steps = 0;
		}
	}
	ctl->steps_done++;
	ctl->bar_count = 0;
	ctl->done_ticket = 0;
	__threadfence();
}

/* ---- kernels ------------------------------------------------------------------ */

/* Norm only (first launch of the split sequence): {sumsq, nonfinite} -> ctl->reduce. */
template <typename GradT>
__global__ void __launch_bounds__(ANNI_THREADS, 4) norm_kernel(const anni_launch a)
{
	__shared__ int s_last;
	double s;

	s = block_sum(norm_phase<GradT>(a));
	if (threadIdx.x == 0) {
		a.ctl->partials[blockIdx.x] = s;
		__threadfence();
		s_last = atomicAdd(&a.ctl->norm_ticket, 1u) == gridDim.x - 1;
	}
	__syncthreads();
	if (s_last) {
		/* last block: every partial is visible; same fixed order as the fused kernel */
		double t;

		__threadfence();
		t = sum_partials(a.ctl, (int)gridDim.x);
		if (threadIdx.x == 0) {
			if (a.flags & ANNI_LAUNCH_ACCUMULATE)	/* a later part of the same shard */
				t += a.ctl->reduce[0];
			a.ctl->reduce[0] = t;
			a.ctl->reduce[1] = isfinite(t) ? 0.0 : 1.0;
			a.ctl->norm_ticket = 0;
		}
	}
}

/*
** ZeRO-1, first half of the step in ONE kernel: the reduce-scatter and the
** norm.  Every rank holds a full gradient arena in peer-accessible memory; this
** rank reads its own shard out of all of them (plain 128-bit loads over NVLink /
** NVSwitch, one per peer in flight per thread), adds them in float in rank
** order, rounds once to the gradient type, writes the reduced shard to local
** memory for the update phase and accumulates the sum of squares of exactly the
** values it wrote.  Result: {sumsq, nonfinite} in the control block, as
** norm_kernel leaves it.  The caller orders this kernel after every rank's
** gradients are complete (a stream-ordered barrier), and all-reduces the two
** doubles afterwards, which also tells every rank that its arena has been read.
*/
/* eight consecutive elements as loaded, not yet widened: keeps many peer loads in flight in few registers */
template <typename T> struct raw8;

template <> struct raw8<__nv_bfloat16> {
	uint4	q;
	__device__ __forceinline__ void load(const void *base, uint64_t e)
	{
		q = __ldcs(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(base) + e));
	}
	__device__ __forceinline__ void load_mc(const void *mc, uint64_t e)
	{
		q = mc_ld_reduce_bf16x8(static_cast<const uint16_t *>(mc) + e);
	}
	static __device__ __forceinline__ void clear(void *base, uint64_t e)
	{
		__stcs(reinterpret_cast<uint4 *>(static_cast<uint16_t *>(base) + e), make_uint4(0, 0, 0, 0));
	}
	__device__ __forceinline__ f32x8 widen() const
	{
		return unpack_bf16x8(q);
	}
};

template <> struct raw8<float> {
	uint4	q[2];
	__device__ __forceinline__ void load(const void *base, uint64_t e)
	{
		const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const float *>(base) + e);

		q[0] = __ldcs(p);
		q[1] = __ldcs(p + 1);
	}
	__device__ __forceinline__ void load_mc(const void *mc, uint64_t e)
	{
		q[0] = mc_ld_reduce_f32x4(static_cast<const float *>(mc) + e);
		q[1] = mc_ld_reduce_f32x4(static_cast<const float *>(mc) + e + 4);
	}
	static __device__ __forceinline__ void clear(void *base, uint64_t e)
	{
		uint4 *p = reinterpret_cast<uint4 *>(static_cast<float *>(base) + e);

		__stcs(p, make_uint4(0, 0, 0, 0));
		__stcs(p + 1, make_uint4(0, 0, 0, 0));
	}
	__device__ __forceinline__ f32x8 widen() const
	{
		f32x8 r;

		r.x[0] = __uint_as_float(q[0].x);
		r.x[1] = __uint_as_float(q[0].y);
		r.x[2] = __uint_as_float(q[0].z);
		r.x[3] = __uint_as_float(q[0].w);
		r.x[4] = __uint_as_float(q[1].x);
		r.x[5] = __uint_as_float(q[1].y);
		r.x[6] = __uint_as_float(q[1].z);
		r.x[7] = __uint_as_float(q[1].w);
		return r;
	}
};

/* sum of one chunk's eight elements over the peers in rank order, rounded to the gradient type, stored, squared */
template <typename GradT, int SLOTS>
__device__ __forceinline__ void reduce_store(const anni_launch &a, const raw8<GradT> (&r)[SLOTS], int first,
	uint64_t e, double &acc0, double &acc1)
{
	f32x8 sum = r[first].widen();

#pragma unroll
	for (int k = 1; k < SLOTS; k++)
		if (k < a.n_peers) {
			const f32x8 x = r[first + k < SLOTS ? first + k : 0].widen();

#pragma unroll
			for (int j = 0; j < ANNI_VEC; j++)
				sum.x[j] = __fadd_rn(sum.x[j], x.x[j]);
		}
	if (sizeof(GradT) == 2)		/* what the update will read back: the rounded value */
		sum = unpack_bf16x8(pack_bf16x8(sum));
	io8<GradT>::store(a.grad, e, sum);
	if (a.own_clear) {		/* this thread's own load of these elements has been consumed above */
		raw8<GradT>::clear(a.own_clear, e);
	}
	norm_accumulate<GradT>(sum, acc0, acc1);
}

/*
** ZeRO-1, first half of the step in ONE kernel: the reduce-scatter and the
** norm.  Every rank holds a full gradient arena in peer-accessible memory; this
** rank reads its own shard out of all of them (plain 128-bit loads over NVLink /
** NVSwitch), adds them in float in rank order, rounds once to the gradient type,
** writes the reduced shard to local memory for the update phase and accumulates
** the sum of squares of exactly the values it wrote.  Result: {sumsq,
** nonfinite} in the control block, as norm_kernel leaves it.  A remote load
** takes a few microseconds, so each thread keeps SLOTS of them in flight
** (peers x consecutive chunks) before it touches the first.  The caller orders
** this kernel after every rank's gradients are complete (a stream-ordered
** barrier) and all-reduces the two doubles afterwards, which also tells every
** rank that its arena has been read.
*/
template <typename GradT>
__global__ void __launch_bounds__(ANNI_THREADS, 4) reduce_norm_kernel(const anni_launch a)
{
	constexpr int SLOTS = sizeof(GradT) == 2 ? 8 : 4;
	__shared__ int s_last;
	const chunk_walk w = walk_init(a.n, a.sc_log2, ANNI_CHUNK_LOG2);
	const uint64_t t8 = (uint64_t)threadIdx.x * ANNI_VEC;
	const int np = a.n_peers;
	const bool pow2 = (np & (np - 1)) == 0 && np <= SLOTS;
	const int lg = np == 1 ? 0 : np == 2 ? 1 : np == 4 ? 2 : 3;
	const int cb = pow2 ? SLOTS >> lg : 0;		/* chunks per batch */
	double acc0 = 0.0;
	double acc1 = 0.0;
	uint64_t it = 0;
	double s;

	if (a.aligned && a.mc_grad) {
		/* in-switch reduction: one multimem load per chunk returns the sum over all ranks */
		for (; it + SLOTS <= w.iters; it += SLOTS) {
			raw8<GradT> r[SLOTS];
			uint64_t cmax = 0;

			for (int ci = 0; ci < SLOTS; ci++)
				cmax = max(cmax, walk_chunk(w, it + ci));
			if ((cmax + 1) * ANNI_CHUNK > a.n)
				break;
#pragma unroll
			for (int sl = 0; sl < SLOTS; sl++)
				r[sl].load_mc(a.mc_grad, walk_chunk(w, it + sl) * ANNI_CHUNK + t8);
#pragma unroll
			for (int sl = 0; sl < SLOTS; sl++) {
				const f32x8 sum = r[sl].widen();
				const uint64_t e = walk_chunk(w, it + sl) * ANNI_CHUNK + t8;

				io8<GradT>::store(a.grad, e, sum);
				norm_accumulate<GradT>(sum, acc0, acc1);
			}
		}
	} else if (a.aligned && cb > 0) {
		for (; it + cb <= w.iters; it += cb) {
			raw8<GradT> r[SLOTS];
			uint64_t cmax = 0;

			for (int ci = 0; ci < cb; ci++)
				cmax = max(cmax, walk_chunk(w, it + ci));
			if ((cmax + 1) * ANNI_CHUNK > a.n)
				break;
#pragma unroll
			for (int sl = 0; sl < SLOTS; sl++)
				r[sl].load(a.peer_grad[sl & (np - 1)], walk_chunk(w, it + (sl >> lg)) * ANNI_CHUNK + t8);
#pragma unroll
			for (int ci = 0; ci < SLOTS; ci++)
				if (ci < cb) {
					if (np == 1)
						reduce_store<GradT, SLOTS>(a, r, ci, walk_chunk(w, it + ci) * ANNI_CHUNK + t8, acc0, acc1);
					else if (np == 2 && ci < SLOTS / 2)
						reduce_store<GradT, SLOTS>(a, r, ci * 2, walk_chunk(w, it + ci) * ANNI_CHUNK + t8, acc0, acc1);
					else if (np == 4 && ci < SLOTS / 4)
						reduce_store<GradT, SLOTS>(a, r, ci * 4, walk_chunk(w, it + ci) * ANNI_CHUNK + t8, acc0, acc1);
					else if (np == 8 && ci < SLOTS / 8)
						reduce_store<GradT, SLOTS>(a, r, 0, walk_chunk(w, it + ci) * ANNI_CHUNK + t8, acc0, acc1);
				}
		}
	}
	for (; it < w.iters; it++) {		/* what is left, chunk by chunk, any peer count */
		const uint64_t c = walk_chunk(w, it);
		const uint64_t e = c * ANNI_CHUNK + t8;

		if (c >= w.chunks)
			continue;
		for (int j = 0; j < ANNI_VEC; j++)
			if (e + j < a.n) {
				float x = io8<GradT>::load1(a.peer_grad[0], e + j);

				for (int k = 1; k < np; k++)
					x = __fadd_rn(x, io8<GradT>::load1(a.peer_grad[k], e + j));
				io8<GradT>::store1(a.grad, e + j, x);
				if (a.own_clear)
					io8<GradT>::store1(a.own_clear, e + j, 0.0f);
				x = io8<GradT>::load1(a.grad, e + j);
				acc0 = fma((double)x, (double)x, acc0);
			}
	}
	s = block_sum(acc0 + acc1);
	if (threadIdx.x == 0) {
		a.ctl->partials[blockIdx.x] = s;
		__threadfence();
		s_last = atomicAdd(&a.ctl->norm_ticket, 1u) == gridDim.x - 1;
	}
	__syncthreads();
	if (s_last) {
		double t;

		__threadfence();
		t = sum_partials(a.ctl, (int)gridDim.x);
		if (threadIdx.x == 0) {
			if (a.flags & ANNI_LAUNCH_ACCUMULATE)	/* a later part of the same shard */
				t += a.ctl->reduce[0];
			a.ctl->reduce[0] = t;
			a.ctl->reduce[1] = isfinite(t) ? 0.0 : 1.0;
			a.ctl->norm_ticket = 0;
		}
	}
}

/* Update only (second launch of the split sequence, or the legacy call with a host multiplier). */
template <typename GradT, typename StateT, bool EXACT, bool ARENA>
__global__ void __launch_bounds__(ANNI_THREADS, 4) update_kernel(const anni_launch a)
{
	decision d;

	if (a.flags & ANNI_LAUNCH_HOST_COEF) {
		d.coef = a.grad_scale;
		d.norm = 0.0;
		d.skip = false;
	} else {
		d = decide(a, a.ctl->reduce[0], a.ctl->reduce[1], a.ctl->loss_scale);
		if (blockIdx.x == 0 && threadIdx.x == 0) {
			a.ctl->norm = d.norm;
			a.ctl->eff_scale = d.coef;
			a.ctl->skipped = d.skip ? 1 : 0;
		}
	}
	update_phase<GradT, StateT, EXACT, ARENA ? MODE_ARENA : MODE_PLAIN>(a, d);
	if (!(a.flags & ANNI_LAUNCH_NO_EPILOGUE))
		step_epilogue(a.ctl, d.skip);
}

/*
** The whole step in one cooperative launch.  PIPE (chosen when some tensor wants an e4m3
** twin): the quantiser follows the update tensor by tensor inside the update phase; block 0
** clears the per-tensor amax and arrival counters before the first barrier, so the step needs
** no memset ahead of it.
*/
template <typename GradT, typename StateT, bool EXACT, bool PIPE>
__global__ void __launch_bounds__(ANNI_THREADS, 4) fused_kernel(const anni_launch a)
{
	decision d;
	double ss = 0.0;
	uint32_t barriers = 0;
	const double loss_scale = a.ctl->loss_scale;

	if (PIPE && blockIdx.x == 0)
		for (int s = threadIdx.x; s < a.n_seg; s += blockDim.x) {
			a.seg_amax[s] = 0.0f;
			a.seg_done[s] = 0u;
		}
	if ((a.flags & ANNI_LAUNCH_NEED_NORM) || PIPE) {
		double s = 0.0;

		if (a.flags & ANNI_LAUNCH_NEED_NORM)
			s = block_sum(norm_phase<GradT>(a));
		if (threadIdx.x == 0)
			a.ctl->partials[blockIdx.x] = s;
		if (!grid_barrier(a.ctl, ++barriers * gridDim.x))
			return;
		if (a.flags & ANNI_LAUNCH_NEED_NORM)
			ss = sum_partials(a.ctl, (int)gridDim.x);
	}
	d = decide(a, ss, 0.0, loss_scale);
	if (blockIdx.x == 0 && threadIdx.x == 0) {
		a.ctl->reduce[0] = ss;
		a.ctl->reduce[1] = isfinite(ss) ? 0.0 : 1.0;
		a.ctl->norm = d.norm;
		a.ctl->eff_scale = d.coef;
		a.ctl->skipped = d.skip ? 1 : 0;
	}
	if (!update_phase<GradT, StateT, EXACT, PIPE ? MODE_PIPE : MODE_PLAIN>(a, d))
		return;
	if (!PIPE && (a.flags & ANNI_LAUNCH_HAS_FP8) && !d.skip) {
		if (!grid_barrier(a.ctl, ++barriers * gridDim.x))
			return;
		quantize_phase(a);
	}
	step_epilogue(a.ctl, d.skip);
}

/* e4m3 twins only (third launch of the split sequence). */
__global__ void __launch_bounds__(ANNI_THREADS, 4) quantize_kernel(const anni_launch a)
{
	if (a.ctl->skipped)
		return;
	quantize_phase(a);
}

/*
** Failure-path self-test: every block arrives at a barrier that expects one
** arrival more than the grid has, so the bounded wait must run out.  Nothing
** faults and nothing hangs: after `max_polls` polls each block records
** ANNI_E_BARRIER_TIMEOUT and returns, exactly as a block of the fused kernel
** would if a peer block never arrived.
*/
__global__ void __launch_bounds__(ANNI_THREADS) barrier_timeout_kernel(anni_control *ctl, uint32_t max_polls)
{
	if (grid_barrier(ctl, gridDim.x + 1, max_polls) && threadIdx.x == 0)
		atomicExch(&ctl->error, ANNI_E_ARG);	/* the barrier must not have opened */
}

/*
** e4m3 twins in the transposed [cols][rows] layout the forward GEMM wants
** (the reference's f32_transpose_to_fp8_kernel, one launch per tensor): here
** one launch for every such tensor.  Tiles of ANNI_TT_R rows x ANNI_TT_C columns of the
** master, dealt round-robin over a persistent grid; tile_prefix[s] = number of tiles
** before tensor s.
**
** A whole, aligned tile (every tile of the LM shapes) goes the fast way: each thread reads
** eight 128-bit pieces of master rows (256 contiguous bytes per tile row), quantises four
** values into one 32-bit word and stores it in shared memory at [row][word ^ swizzle]; then
** eight lanes gather one 128-byte row of the transposed tile, 16 bytes each, and store it
** with one 128-bit access.  The swizzle (word index XOR 2 * (row / 16)) keeps both the
** row-wise stores and the column-wise gathers free of bank conflicts.  Edge tiles and
** unaligned tensors go element by element.
*/
__global__ void __launch_bounds__(ANNI_THREADS) quantize_transposed_kernel(const anni_launch a,
	const int64_t *tile_prefix, int64_t n_tiles)
{
	__shared__ uint32_t tile[ANNI_TT_R * (ANNI_TT_C / 4)];	/* 128 rows x 16 words of four e4m3 codes */
	uint8_t *tile_b = reinterpret_cast<uint8_t *>(tile);		/* the same bytes, unswizzled, for edge tiles */
	const int tid = threadIdx.x;
	int seg = 0;

	if (a.ctl->skipped)
		return;
	if (blockIdx.x == 0)
		for (int s = threadIdx.x; s < a.n_seg; s += blockDim.x)
			if ((a.seg_flags[s] & ANNI_SEG_TWIN_FP8) && a.seg_aux[s].fp8_t_off >= 0)
				a.seg_scale[s] = fp8_scale(a.seg_amax[s]);
	for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
		while (seg + 1 < a.n_seg && tile_prefix[seg + 1] <= t)
			seg++;
		const anni_seg_derived ax = a.seg_aux[seg];
		const int tiles_x = (ax.cols + ANNI_TT_C - 1) / ANNI_TT_C;
		const int64_t lt = t - tile_prefix[seg];
		const int r0 = (int)(lt / tiles_x) * ANNI_TT_R;
		const int c0 = (int)(lt % tiles_x) * ANNI_TT_C;
		const float inv = __fdiv_rn(1.0f, fp8_scale(a.seg_amax[seg]));
		const float *src = a.master + ((uint64_t)a.seg_off[seg] - a.arena_off);
		uint8_t *dst = a.fp8_t + ax.fp8_t_off;
		const bool fast = r0 + ANNI_TT_R <= ax.rows && c0 + ANNI_TT_C <= ax.cols && (ax.cols & 3) == 0
		    && (ax.rows & 15) == 0 && ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0;

		if (fast) {
			const float *s0 = src + (uint64_t)r0 * ax.cols + c0;

#pragma unroll
			for (int half = 0; half < 2; half++) {
				f32x4 v[4];

#pragma unroll
				for (int i = 0; i < 4; i++) {
					const int f = tid + ANNI_THREADS * (half * 4 + i);	/* 128-bit piece of the tile */

					v[i] = io4<float>::load(s0 + (uint64_t)(f >> 4) * ax.cols, (uint64_t)(f & 15) * 4);
				}
#pragma unroll
				for (int i = 0; i < 4; i++) {
					const int f = tid + ANNI_THREADS * (half * 4 + i);
					const int r = f >> 4;

					tile[r * 16 + ((f & 15) ^ (((r >> 4) & 7) << 1))] = e4m3x4(v[i], inv);
				}
			}
			__syncthreads();
#pragma unroll
			for (int j = 0; j < 2; j++) {
				const int id = tid + ANNI_THREADS * j;	/* 16-byte piece of the transposed tile */
				const int c = id >> 3;			/* source column = destination row */
				const int sg = id & 7;			/* source rows 16 sg .. 16 sg + 15 */
				const int w = (c >> 2) ^ (sg << 1);
				const uint32_t sel = (uint32_t)(c & 3) | ((4u + (uint32_t)(c & 3)) << 4);
				uint32_t out[4];

#pragma unroll
				for (int k = 0; k < 4; k++) {
					const uint32_t *row = &tile[(16 * sg + 4 * k) * 16 + w];
					const uint32_t lo = __byte_perm(row[0], row[16], sel);	/* the column's byte of two rows */
					const uint32_t hi = __byte_perm(row[32], row[48], sel);

					out[k] = __byte_perm(lo, hi, 0x5410);
				}
				__stcs(reinterpret_cast<uint4 *>(dst + (uint64_t)(c0 + c) * ax.rows + r0 + 16 * sg),
				    make_uint4(out[0], out[1], out[2], out[3]));
			}
			__syncthreads();
			continue;
		}
		for (int i = tid; i < ANNI_TT_R * ANNI_TT_C; i += ANNI_THREADS) {
			const int r = i / ANNI_TT_C;
			const int c = i % ANNI_TT_C;

			if (r0 + r < ax.rows && c0 + c < ax.cols)
				tile_b[i] = (uint8_t)__nv_cvt_float_to_fp8(
				    src[(uint64_t)(r0 + r) * ax.cols + c0 + c] * inv, __NV_SATFINITE, __NV_E4M3);
		}
		__syncthreads();
		/* now consecutive threads walk the rows of the source (contiguous in the transposed destination) */
		for (int i = tid; i < ANNI_TT_R * ANNI_TT_C; i += ANNI_THREADS) {
			const int c = i / ANNI_TT_R;
			const int r = i % ANNI_TT_R;

			if (c0 + c < ax.cols && r0 + r < ax.rows)
				dst[(uint64_t)(c0 + c) * ax.rows + r0 + r] = tile_b[r * ANNI_TT_C + c];
		}
		__syncthreads();
	}
}

/*
** ZeRO-1: what the update's own walk cannot reach of a rank's full gradient arena -- elements
** [from, stride) of every part, when this rank's shard is shorter than the others' (the last
** rank, or a rank without elements).  Usually a few thousand elements.
*/
template <typename T>
__global__ void __launch_bounds__(ANNI_THREADS) zero_tail_kernel(T *arena, uint64_t from, uint64_t stride,
	int parts)
{
	const uint64_t len = stride - from;
	const uint64_t total = len * (uint64_t)parts;

	for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
	    i += (uint64_t)gridDim.x * blockDim.x)
		arena[(i / len) * stride + from + i % len] = 0;
}

/* One-shot fp32 -> bf16 of a flat buffer (seeding the twin; num/gpu.h:73 of the reference). */
__global__ void __launch_bounds__(ANNI_THREADS) f32_to_bf16_kernel(uint16_t *dst, const float *src,
	uint64_t n, int aligned)
{
	const uint64_t stride = (uint64_t)gridDim.x * ANNI_CHUNK;

	for (uint64_t e = (uint64_t)blockIdx.x * ANNI_CHUNK + (uint64_t)threadIdx.x * ANNI_VEC; e < n;
	    e += stride) {
		if (aligned && e + ANNI_VEC <= n)
			io8<__nv_bfloat16>::store(dst, e, io8<float>::load(src, e));
		else
			for (int k = 0; k < ANNI_VEC && e + k < n; k++)
				io8<__nv_bfloat16>::store1(dst, e + k, src[e + k]);
	}
}

/* y += a x (num/gpu.h:299 of the reference, gpu_mat_axpy). */
__global__ void __launch_bounds__(ANNI_THREADS) axpy_kernel(float *y, const float *x, float a,
	uint64_t n, int aligned)
{
	const uint64_t stride = (uint64_t)gridDim.x * ANNI_UCHUNK;

	for (uint64_t e = (uint64_t)blockIdx.x * ANNI_UCHUNK + (uint64_t)threadIdx.x * ANNI_UVEC; e < n;
	    e += stride) {
		if (aligned && e + ANNI_UVEC <= n) {
			const f32x4 xv = io4<float>::load(x, e);
			f32x4 yv = io4<float>::load(y, e);

#pragma unroll
			for (int k = 0; k < ANNI_UVEC; k++)
				yv.x[k] = fmaf(a, xv.x[k], yv.x[k]);
			io4<float>::store(y, e, yv);
		} else
			for (int k = 0; k < ANNI_UVEC && e + k < n; k++)
				y[e + k] = fmaf(a, x[e + k], y[e + k]);
	}
}

std::atomic<uint64_t> g_launches{0};

template <typename K> int occupancy_blocks(K kernel)
{
	int dev = 0;
	int sms = 0;
	int per_sm = 0;

	if (cudaGetDevice(&dev) != cudaSuccess
	    || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess
	    || cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, ANNI_THREADS, 0)
	    != cudaSuccess || sms <= 0 || per_sm <= 0)
		return -1;
	int blocks = sms * per_sm;

	return blocks > ANNI_MAX_BLOCKS ? ANNI_MAX_BLOCKS / sms * sms : blocks;
}

template <typename GradT, typename StateT>
int launch_update_t(const anni_launch *a, int blocks, cudaStream_t st)
{
	const bool arena = a->zero_parts > 0;	/* a full gradient arena to clear instead of the bound buffer */

	if (a->flags & ANNI_STEP_EXACT_UPDATE) {
		if (arena)
			update_kernel<GradT, StateT, true, true><<<blocks, ANNI_THREADS, 0, st>>>(*a);
		else
			update_kernel<GradT, StateT, true, false><<<blocks, ANNI_THREADS, 0, st>>>(*a);
	} else if (arena)
		update_kernel<GradT, StateT, false, true><<<blocks, ANNI_THREADS, 0, st>>>(*a);
	else
		update_kernel<GradT, StateT, false, false><<<blocks, ANNI_THREADS, 0, st>>>(*a);
	return cudaGetLastError() == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}

template <typename GradT, typename StateT>
int launch_fused_t(const anni_launch *a, int blocks, cudaStream_t st)
{
	void *args[] = { (void *)a };
	const bool pipe = (a->flags & ANNI_LAUNCH_FP8_PIPE) && (a->flags & ANNI_LAUNCH_HAS_FP8);
	const void *k = (a->flags & ANNI_STEP_EXACT_UPDATE)
	    ? (pipe ? (const void *)fused_kernel<GradT, StateT, true, true>
	    : (const void *)fused_kernel<GradT, StateT, true, false>)
	    : (pipe ? (const void *)fused_kernel<GradT, StateT, false, true>
	    : (const void *)fused_kernel<GradT, StateT, false, false>);

	return cudaLaunchCooperativeKernel(k, dim3(blocks), dim3(ANNI_THREADS), args, 0, st)
	    == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}

/* resident blocks of the heaviest variant: every variant then runs with the same grid */
template <typename GradT, typename StateT> int grid_t(int cooperative)
{
	int best = cooperative ? occupancy_blocks(fused_kernel<GradT, StateT, true, false>)
	    : occupancy_blocks(update_kernel<GradT, StateT, true, true>);
	const int others[3] = {
		cooperative ? occupancy_blocks(fused_kernel<GradT, StateT, false, false>)
		    : occupancy_blocks(update_kernel<GradT, StateT, false, true>),
		cooperative ? occupancy_blocks(fused_kernel<GradT, StateT, true, true>) : best,
		cooperative ? occupancy_blocks(fused_kernel<GradT, StateT, false, true>) : best,
	};

	for (int k = 0; k < 3; k++)
		if (others[k] < best)
			best = others[k];
	return best;
}

/*
** How many of the `blocks` resident blocks to launch.  With fp32 moments a thread has more
** bytes in flight per chunk, and four resident blocks per SM then queue more loads than the
** memory system digests at its best rate: three per SM measured 3-6 % faster (one GPU,
** 185 M and 555 M parameters), except where the double-precision update term keeps the
** blocks busy for longer (bf16 gradients, exact update), which needs all four.  Both forms
** of the step ask with the same arguments, so their grids and block partials agree.
*/
int tuned_blocks(int blocks, int grad_dtype, int state_dtype, int flags)
{
	int dev = 0;
	int sms = 0;

	if (state_dtype != ANNI_DT_F32)
		return blocks;
	if ((flags & ANNI_STEP_EXACT_UPDATE) && grad_dtype != ANNI_DT_F32)
		return blocks;
	if (cudaGetDevice(&dev) != cudaSuccess
	    || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
		return blocks;
	return blocks == 4 * sms ? 3 * sms : blocks;	/* an explicit smaller grid (tuning knob) is left alone */
}

}	/* namespace */

extern "C" void anni_count_launch(void)
{
	g_launches.fetch_add(1, std::memory_order_relaxed);
}

extern "C" uint64_t anni_kernel_launches(void)
{
	return g_launches.load(std::memory_order_relaxed);
}

extern "C" int anni_grid_blocks(int grad_dtype, int state_dtype, int cooperative)
{
	const bool gb = grad_dtype == ANNI_DT_BF16;
	const bool sb = state_dtype == ANNI_DT_BF16;

	if (gb && sb)
		return grid_t<__nv_bfloat16, __nv_bfloat16>(cooperative);
	if (gb)
		return grid_t<__nv_bfloat16, float>(cooperative);
	if (sb)
		return grid_t<float, __nv_bfloat16>(cooperative);
	return grid_t<float, float>(cooperative);
}

/*
** Host side of the arithmetic contract: everything that depends only on the
** step's scalars is computed once, in double, and rounded once.  Rejections
** are those of the reference launcher (num/gpu_cuda.cu:8675-8682): lr <= 0,
** t < 1, a bias correction that is not positive.
*/
extern "C" int anni_fill_hyper(anni_launch *a, const anni_optstep_hyper *hp)
{
	double bc1;
	double bc2;

	if (!a || !hp || !(hp->lr > 0.0) || hp->t < 1)
		return ANNI_E_ARG;
	bc1 = 1.0 - pow(hp->beta1, (double)hp->t);
	bc2 = 1.0 - pow(hp->beta2, (double)hp->t);
	if (!(bc1 > 0.0) || !(bc2 > 0.0))
		return ANNI_E_ARG;
	a->grad_scale = hp->grad_scale;
	a->clip = hp->grad_clip > 0.0 ? hp->grad_clip : 0.0;
	a->b1 = hp->beta1;
	a->omb1 = 1.0 - hp->beta1;
	a->b2 = hp->beta2;
	a->omb2 = 1.0 - hp->beta2;
	a->lrbc1 = (float)(hp->lr / bc1);
	a->lrbc1d = hp->lr / bc1;
	a->lrwdd = hp->weight_decay > 0.0 ? hp->lr * hp->weight_decay : 0.0;
	a->ibc2d = 1.0 / bc2;
	a->epsd = hp->eps;
	a->ibc2 = (float)(1.0 / bc2);
	a->eps = (float)hp->eps;
	/* the same three floats at the binary scales the fast update works in (exact products) */
	a->ibc2_s24 = a->ibc2 * 16777216.0f;
	a->eps_s40 = a->eps * 1099511627776.0f;
	a->lrbc1_s40 = a->lrbc1 * 1099511627776.0f;
	if (!isfinite(a->ibc2_s24) || !isfinite(a->eps_s40) || !isfinite(a->lrbc1_s40))
		return ANNI_E_ARG;
	a->lrwd = hp->weight_decay > 0.0 ? (float)(hp->lr * hp->weight_decay) : 0.0f;
	a->flags = (a->flags & ~0xff) | (hp->flags & 0xff);
	if (a->clip > 0.0 || (hp->flags & ANNI_STEP_CHECK_FINITE))
		a->flags |= ANNI_LAUNCH_NEED_NORM;
	else
		a->flags &= ~ANNI_LAUNCH_NEED_NORM;
	return ANNI_OK;
}

extern "C" int anni_launch_norm(const anni_launch *a, int grad_dtype, int state_dtype, int blocks,
	cudaStream_t st)
{
	if (!a || blocks < 1 || blocks > ANNI_MAX_BLOCKS)
		return ANNI_E_ARG;
	blocks = tuned_blocks(blocks, grad_dtype, state_dtype, a->flags);
	if (grad_dtype == ANNI_DT_BF16)
		norm_kernel<__nv_bfloat16><<<blocks, ANNI_THREADS, 0, st>>>(*a);
	else
		norm_kernel<float><<<blocks, ANNI_THREADS, 0, st>>>(*a);
	anni_count_launch();
	return cudaGetLastError() == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}

extern "C" int anni_launch_reduce_norm(const anni_launch *a, int grad_dtype, int blocks, cudaStream_t st)
{
	if (!a || blocks < 1 || blocks > ANNI_MAX_BLOCKS || a->n_peers < 1 || a->n_peers > ANNI_MAX_PEERS)
		return ANNI_E_ARG;
	if (grad_dtype == ANNI_DT_BF16)
		reduce_norm_kernel<__nv_bfloat16><<<blocks, ANNI_THREADS, 0, st>>>(*a);
	else
		reduce_norm_kernel<float><<<blocks, ANNI_THREADS, 0, st>>>(*a);
	anni_count_launch();
	return cudaGetLastError() == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}

extern "C" int anni_launch_zero_tail(void *arena, int grad_dtype, uint64_t from, uint64_t stride, int parts,
	cudaStream_t st)
{
	uint64_t total;
	int blocks;

	if (!arena || from > stride || parts < 1)
		return ANNI_E_ARG;
	total = (stride - from) * (uint64_t)parts;
	if (total == 0)
		return ANNI_OK;
	blocks = (int)((total + ANNI_THREADS - 1) / ANNI_THREADS < 4096 ? (total + ANNI_THREADS - 1) / ANNI_THREADS : 4096);
	if (grad_dtype == ANNI_DT_BF16)
		zero_tail_kernel<uint16_t><<<blocks, ANNI_THREADS, 0, st>>>((uint16_t *)arena, from, stride, parts);
	else
		zero_tail_kernel<uint32_t><<<blocks, ANNI_THREADS, 0, st>>>((uint32_t *)arena, from, stride, parts);
	anni_count_launch();
	return cudaGetLastError() == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}

extern "C" int anni_launch_update(const anni_launch *a, int grad_dtype, int state_dtype, int blocks,
	cudaStream_t st)
{
	const bool gb = grad_dtype == ANNI_DT_BF16;
	const bool sb = state_dtype == ANNI_DT_BF16;

	if (!a || blocks < 1 || blocks > ANNI_MAX_BLOCKS)
		return ANNI_E_ARG;
	blocks = tuned_blocks(blocks, grad_dtype, state_dtype, a->flags);
	anni_count_launch();
	if (gb && sb)
		return launch_update_t<__nv_bfloat16, __nv_bfloat16>(a, blocks, st);
	if (gb)
		return launch_update_t<__nv_bfloat16, float>(a, blocks, st);
	if (sb)
		return launch_update_t<float, __nv_bfloat16>(a, blocks, st);
	return launch_update_t<float, float>(a, blocks, st);
}

extern "C" int anni_launch_fused(const anni_launch *a, int grad_dtype, int state_dtype, int blocks,
	cudaStream_t st)
{
	const bool gb = grad_dtype == ANNI_DT_BF16;
	const bool sb = state_dtype == ANNI_DT_BF16;

	if (!a || blocks < 1 || blocks > ANNI_MAX_BLOCKS)
		return ANNI_E_ARG;
	blocks = tuned_blocks(blocks, grad_dtype, state_dtype, a->flags);
	anni_count_launch();
	if (gb && sb)
		return launch_fused_t<__nv_bfloat16, __nv_bfloat16>(a, blocks, st);
	if (gb)
		return launch_fused_t<__nv_bfloat16, float>(a, blocks, st);
	if (sb)
		return launch_fused_t<float, __nv_bfloat16>(a, blocks, st);
	return launch_fused_t<float, float>(a, blocks, st);
}

extern "C" int anni_launch_quantize_transposed(const anni_launch *a, const int64_t *tile_prefix,
	int64_t n_tiles, int blocks, cudaStream_t st)
{
	if (!a || !tile_prefix || !a->seg_aux || !a->fp8_t || blocks < 1)
		return ANNI_E_ARG;
	if (n_tiles <= 0)
		return ANNI_OK;
	quantize_transposed_kernel<<<blocks, ANNI_THREADS, 0, st>>>(*a, tile_prefix, n_tiles);
	anni_count_launch();
	return cudaGetLastError() == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}

extern "C" int anni_launch_barrier_timeout(anni_control *ctl, int blocks, unsigned max_polls, cudaStream_t st)
{
	if (!ctl || blocks < 1 || blocks > ANNI_MAX_BLOCKS || max_polls > ANNI_WAIT_POLLS)
		return ANNI_E_ARG;
	barrier_timeout_kernel<<<blocks, ANNI_THREADS, 0, st>>>(ctl, max_polls);
	anni_count_launch();
	return cudaGetLastError() == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}

extern "C" int anni_launch_quantize(const anni_launch *a, int blocks, cudaStream_t st)
{
	if (!a || blocks < 1 || blocks > ANNI_MAX_BLOCKS)
		return ANNI_E_ARG;
	quantize_kernel<<<blocks, ANNI_THREADS, 0, st>>>(*a);
	anni_count_launch();
	return cudaGetLastError() == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}

static int flat_blocks(uint64_t n)
{
	int dev = 0;
	int sms = 148;
	uint64_t want = (n + ANNI_CHUNK - 1) / ANNI_CHUNK;

	if (cudaGetDevice(&dev) == cudaSuccess)
		cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
	if (want > (uint64_t)sms * 8)
		want = (uint64_t)sms * 8;
	return want < 1 ? 1 : (int)want;
}

extern "C" int anni_launch_f32_to_bf16(uint16_t *dst, const float *src, uint64_t n, cudaStream_t st)
{
	const int aligned = (((uintptr_t)dst | (uintptr_t)src) & 15) == 0;

	if (!dst || !src || n == 0)
		return ANNI_E_ARG;
	f32_to_bf16_kernel<<<flat_blocks(n), ANNI_THREADS, 0, st>>>(dst, src, n, aligned);
	anni_count_launch();
	return cudaGetLastError() == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}

extern "C" int anni_launch_axpy(float *y, const float *x, float a, uint64_t n, cudaStream_t st)
{
	if (!y || !x || n == 0)
		return ANNI_E_ARG;
	axpy_kernel<<<flat_blocks(n), ANNI_THREADS, 0, st>>>(y, x, a, n,
	    (((uintptr_t)y | (uintptr_t)x) & 15) == 0);
	anni_count_launch();
	return cudaGetLastError() == cudaSuccess ? ANNI_OK : ANNI_E_CUDA;
}
