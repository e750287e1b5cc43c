/*
** TEST INFRASTRUCTURE, not product code: CPU restatement of the reference's
** optimizer-step path.  See oracle_adam.c for what each function follows.
*/
#ifndef ORACLE_ADAM_H__
#define ORACLE_ADAM_H__

#include <stdint.h>

#define ORACLE_DT_F32	0
#define ORACLE_DT_BF16	1

/* per-segment flags (same bit meaning as the product's segment table) */
#define ORACLE_SEG_WD		1u	/* decoupled weight decay applies */
#define ORACLE_SEG_TWIN_BF16	2u
#define ORACLE_SEG_TWIN_FP8	4u

typedef struct oracle_step_args {
	int64_t	n;
	float	*param;		/* fp32 master, updated in place */
	void	*grad;		/* fp32 or bf16 (uint16), zeroed by the step */
	void	*m;		/* fp32 or bf16 storage */
	void	*v;
	int	grad_dtype;
	int	state_dtype;
	int	n_seg;		/* 0: one implicit segment, wd on */
	const int64_t	*seg_off;	/* n_seg + 1 element offsets */
	const uint32_t	*seg_flags;
	double	lr;
	double	beta1;
	double	beta2;
	double	eps;
	double	weight_decay;
	double	grad_clip;	/* 0 = off */
	double	grad_scale;	/* 1/(batch) * 1/loss_scale, folded */
	int	t_before;	/* opt->t before the call */
	int	check_finite;	/* device-path skip rule even when grad_clip == 0 */
	int	zero_grad;	/* the reference always zeroes; 0 only for variants */
	/* outputs */
	double	norm;		/* sqrt(sum (g*grad_scale)^2), before clipping */
	double	eff_scale;	/* grad_scale after clipping */
	int	skipped;
	int	t_after;
} oracle_step_args;

uint16_t oracle_bf16_rne(float x);
float	oracle_bf16_to_f32(uint16_t h);
uint8_t	oracle_fp8_e4m3_satfinite(float x);
float	oracle_fp8_e4m3_to_f32(uint8_t q);

double	oracle_sumsq(const void *grad, int dtype, int64_t n, double scale);
int	oracle_adam_step(oracle_step_args *a);
void	oracle_twin_bf16(const float *param, int64_t n, uint16_t *out);
void	oracle_fp8_tensor_quant(const float *param, int64_t n, float *amax_out,
		float *scale_out, uint8_t *q_out);
double	oracle_lr_schedule(double base_lr, int step, int warmup, int decay,
		const char *kind, int from);

typedef struct oracle_loss_scaler {
	double	scale;
	int	good_steps;
	int	growth_interval;
	double	growth;
	double	backoff;
	double	min_scale;
	double	max_scale;
} oracle_loss_scaler;
void	oracle_loss_scale_update(oracle_loss_scaler *s, int skipped);

int	oracle_ckpt_write_adam(const char *path, int append, int epoch, int step,
		int t, int64_t n, const float *m, const float *v);
int	oracle_ckpt_read_adam(const char *path, int64_t trailer_off, int *epoch,
		int *step, int *t, int64_t *n, float *m, float *v, int64_t cap);

#endif
