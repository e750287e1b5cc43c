/*
** Whole checkpoints in the reference's format (lang/lm_serialize.c of the
** reference project), read into / written from the optimizer's flat order, so
** that a checkpoint of the reference trainer resumes on this engine and the
** other way round.  Host code only.
**
** File layout (little-endian, as the reference writes it on x86-64):
**   int32 magic  LMCF 0x46434D4C (byte-level model) | LMCV 0x56434D4C (BPE table
**                embedded) | LMCT 0x54434D4C (BPE + tied embedding)      :103-106
**   int32 sizeof(real) = 4, d_model, n_heads, d_ff, max_ctx, n_blocks, vocab   :107-110
**   [LMCV/LMCT] int32 n_merges (| 0x40000000 flag), n_merges x {int32 left, right}  (lang/bpe.c:383-401)
**   [untied]    embedding table  V x D                                   :113-114
**   per block   wq wk wv wo (D x D), w1 (D x FF), b1 (FF), w2 (FF x D), b2 (D),
**               ln1.gamma ln1.beta ln2.gamma ln2.beta (D)                :79-91
**   w_head (D x V), b_head (V)                                           :121-122
**   each matrix as int32 rows, cols, data; each vector as int32 n, data  :30-66
**   int32 has_adam; if 1: epoch, step, t, n, then n x (m, v)             :316-319, :263-296
** The optimizer's order (lang/lm_adam.c:117-136) differs: w_head, b_head,
** [embedding], then the blocks.  Files are written to PATH.tmp and renamed.
*/
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "anni_lm_adam.h"

#define MAGIC_F	0x46434D4C
#define MAGIC_V	0x56434D4C
#define MAGIC_T	0x54434D4C
#define MERGE_FLAG	0x40000000
#define MAX_MERGES	(1 << 22)

namespace {

int rd32(FILE *fp, int32_t *v)
{
	return fread(v, 4, 1, fp) == 1 ? 0 : -1;
}

int wr32(FILE *fp, int32_t v)
{
	return fwrite(&v, 4, 1, fp) == 1 ? 0 : -1;
}

/* one tensor of the file: where it sits in the optimizer's flat order */
struct tensor_ref {
	int64_t	off;
	int	rows;
	int	cols;	/* 0: a vector of `rows` elements */
};

/* the tensors in FILE order with their offsets in OPTIMIZER order; returns the count */
int file_order(const anni_ckpt_model *k, tensor_ref *out, int64_t *n_out)
{
	const int64_t D = k->d_model;
	const int64_t FF = k->d_ff;
	const int64_t V = k->vocab;
	int64_t off = 0;
	int64_t head_off;
	int64_t bhead_off;
	int64_t embed_off = -1;
	int cnt = 0;

	head_off = off;
	off += D * V;
	bhead_off = off;
	off += V;
	if (!k->tied) {
		embed_off = off;
		off += V * D;
		out[cnt++] = { embed_off, (int)V, (int)D };
	}
	for (int b = 0; b < k->n_blocks; b++) {
		for (int q = 0; q < 4; q++) {
			out[cnt++] = { off, (int)D, (int)D };
			off += D * D;
		}
		out[cnt++] = { off, (int)D, (int)FF };
		off += D * FF;
		out[cnt++] = { off, (int)FF, 0 };
		off += FF;
		out[cnt++] = { off, (int)FF, (int)D };
		off += FF * D;
		out[cnt++] = { off, (int)D, 0 };
		off += D;
		for (int q = 0; q < 4; q++) {
			out[cnt++] = { off, (int)D, 0 };
			off += D;
		}
	}
	out[cnt++] = { head_off, (int)D, (int)V };
	out[cnt++] = { bhead_off, (int)V, 0 };
	*n_out = off;
	return cnt;
}

int read_header(FILE *fp, anni_ckpt_model *k)
{
	int32_t magic;
	int32_t real_size;
	int32_t v[6];

	memset(k, 0, sizeof(*k));
	if (rd32(fp, &magic) != 0 || rd32(fp, &real_size) != 0 || real_size != 4)
		return -1;
	if (magic == MAGIC_F)
		k->kind = 0;
	else if (magic == MAGIC_V)
		k->kind = 1;
	else if (magic == MAGIC_T)
		k->kind = 2;
	else
		return -1;	/* includes the legacy double-precision magic, as the reference rejects it */
	for (int i = 0; i < 6; i++)
		if (rd32(fp, &v[i]) != 0)
			return -1;
	k->d_model = v[0];
	k->n_heads = v[1];
	k->d_ff = v[2];
	k->max_ctx = v[3];
	k->n_blocks = v[4];
	k->vocab = v[5];
	k->tied = k->kind == 2;
	if (k->d_model <= 0 || k->d_ff <= 0 || k->n_blocks < 0 || k->vocab <= 0 || k->n_blocks > 4096)
		return -1;
	if (k->kind != 0) {
		int32_t raw;

		if (rd32(fp, &raw) != 0 || raw < 0 || (raw & ~MERGE_FLAG) > MAX_MERGES)
			return -1;
		k->merges_word = raw;
		k->n_merges = raw & ~MERGE_FLAG;
	}
	return 0;
}

}	/* namespace */

extern "C" int anni_ckpt_probe(const char *path, anni_ckpt_model *k)
{
	FILE *fp;
	tensor_ref *tr;
	int64_t n = 0;
	int cnt;
	int rc = ANNI_E_ARG;
	int32_t h[5];

	if (!path || !k)
		return ANNI_E_ARG;
	fp = fopen(path, "rb");
	if (!fp)
		return ANNI_E_ARG;
	if (read_header(fp, k) != 0) {
		fclose(fp);
		return ANNI_E_ARG;
	}
	tr = (tensor_ref *)malloc((size_t)(3 + 12 * k->n_blocks) * sizeof(tensor_ref));
	if (!tr) {
		fclose(fp);
		return ANNI_E_NOMEM;
	}
	cnt = file_order(k, tr, &n);
	k->n = n;
	/* skip the merge table and the tensors, then look at the Adam header */
	if (fseek(fp, (long)k->n_merges * 8, SEEK_CUR) == 0) {
		int ok = 1;

		for (int i = 0; i < cnt && ok; i++) {
			const int64_t elems = tr[i].cols ? (int64_t)tr[i].rows * tr[i].cols : tr[i].rows;

			if (fseek(fp, (tr[i].cols ? 8 : 4) + (long)(elems * 4), SEEK_CUR) != 0)
				ok = 0;
		}
		if (ok && rd32(fp, &h[0]) == 0) {
			k->has_adam = h[0] == 1;
			rc = ANNI_OK;
			if (k->has_adam) {
				if (rd32(fp, &h[1]) != 0 || rd32(fp, &h[2]) != 0 || rd32(fp, &h[3]) != 0
				    || rd32(fp, &h[4]) != 0 || (int64_t)h[4] != n)
					rc = ANNI_E_ARG;	/* slot count must match the model (lm_serialize.c:562) */
				k->epoch = h[1];
				k->step = h[2];
				k->t = h[3];
			}
		}
	}
	free(tr);
	fclose(fp);
	return rc;
}

extern "C" int anni_ckpt_load(const char *path, anni_ckpt_model *k, float *w, float *m, float *v,
	int32_t *merges)
{
	FILE *fp;
	tensor_ref *tr;
	int64_t n = 0;
	int cnt;
	int rc = ANNI_E_ARG;
	int32_t h[5];

	if (!path || !k || !w)
		return ANNI_E_ARG;
	fp = fopen(path, "rb");
	if (!fp)
		return ANNI_E_ARG;
	if (read_header(fp, k) != 0) {
		fclose(fp);
		return ANNI_E_ARG;
	}
	tr = (tensor_ref *)malloc((size_t)(3 + 12 * k->n_blocks) * sizeof(tensor_ref));
	if (!tr) {
		fclose(fp);
		return ANNI_E_NOMEM;
	}
	cnt = file_order(k, tr, &n);
	k->n = n;
	if (k->n_merges > 0) {
		if (merges) {
			if (fread(merges, 8, (size_t)k->n_merges, fp) != (size_t)k->n_merges)
				goto out;
		} else if (fseek(fp, (long)k->n_merges * 8, SEEK_CUR) != 0)
			goto out;
	}
	for (int i = 0; i < cnt; i++) {
		const int64_t elems = tr[i].cols ? (int64_t)tr[i].rows * tr[i].cols : tr[i].rows;
		int32_t a;
		int32_t b = 0;

		/* shapes are checked against the header's dimensions, as read_mat_into does (:41-52) */
		if (rd32(fp, &a) != 0 || a != tr[i].rows || (tr[i].cols && (rd32(fp, &b) != 0 || b != tr[i].cols)))
			goto out;
		if (fread(w + tr[i].off, 4, (size_t)elems, fp) != (size_t)elems)
			goto out;
	}
	if (rd32(fp, &h[0]) != 0)
		h[0] = 0;		/* a weights-only file may simply end here (lm_load, :227) */
	k->has_adam = h[0] == 1;
	if (k->has_adam) {
		float pair[2];

		if (rd32(fp, &h[1]) != 0 || rd32(fp, &h[2]) != 0 || rd32(fp, &h[3]) != 0
		    || rd32(fp, &h[4]) != 0 || (int64_t)h[4] != n)
			goto out;
		k->epoch = h[1];
		k->step = h[2];
		k->t = h[3];
		if (m && v) {
			float *buf = (float *)malloc((size_t)(1 << 21) * 2 * sizeof(float));

			if (!buf)
				goto out;
			for (int64_t i = 0; i < n; ) {
				const int64_t c = n - i < (1 << 21) ? n - i : (1 << 21);

				if (fread(buf, 8, (size_t)c, fp) != (size_t)c) {
					free(buf);
					goto out;
				}
				for (int64_t j = 0; j < c; j++) {
					m[i + j] = buf[2 * j];
					v[i + j] = buf[2 * j + 1];
				}
				i += c;
			}
			free(buf);
		}
		(void)pair;
	}
	rc = ANNI_OK;
out:
	free(tr);
	fclose(fp);
	return rc;
}

extern "C" int anni_ckpt_save(const char *path, const anni_ckpt_model *k, const int32_t *merges,
	const float *w, const float *m, const float *v)
{
	char tmp[1024];
	FILE *fp;
	tensor_ref *tr;
	int64_t n = 0;
	int cnt;
	int bad = 0;
	static const int32_t magic[3] = { MAGIC_F, MAGIC_V, MAGIC_T };

	if (!path || !k || !w || k->kind < 0 || k->kind > 2 || (k->kind != 0 && k->n_merges > 0 && !merges)
	    || (k->tied != 0) != (k->kind == 2))
		return ANNI_E_ARG;
	if (snprintf(tmp, sizeof(tmp), "%s.tmp", path) >= (int)sizeof(tmp))
		return ANNI_E_ARG;
	tr = (tensor_ref *)malloc((size_t)(3 + 12 * k->n_blocks) * sizeof(tensor_ref));
	if (!tr)
		return ANNI_E_NOMEM;
	cnt = file_order(k, tr, &n);
	if (n > 0x7fffffff) {
		free(tr);
		return ANNI_E_LIMIT;	/* the format counts slots in an int32 */
	}
	fp = fopen(tmp, "wb");
	if (!fp) {
		free(tr);
		return ANNI_E_ARG;
	}
	bad |= wr32(fp, magic[k->kind]) | wr32(fp, 4) | wr32(fp, k->d_model) | wr32(fp, k->n_heads)
	    | wr32(fp, k->d_ff) | wr32(fp, k->max_ctx) | wr32(fp, k->n_blocks) | wr32(fp, k->vocab);
	if (k->kind != 0) {
		bad |= wr32(fp, k->merges_word ? k->merges_word : k->n_merges);
		if (k->n_merges > 0 && fwrite(merges, 8, (size_t)k->n_merges, fp) != (size_t)k->n_merges)
			bad = 1;
	}
	for (int i = 0; i < cnt && !bad; i++) {
		const int64_t elems = tr[i].cols ? (int64_t)tr[i].rows * tr[i].cols : tr[i].rows;

		bad |= wr32(fp, tr[i].rows);
		if (tr[i].cols)
			bad |= wr32(fp, tr[i].cols);
		if (fwrite(w + tr[i].off, 4, (size_t)elems, fp) != (size_t)elems)
			bad = 1;
	}
	free(tr);
	if (!bad && m && v) {
		if (fclose(fp) != 0)
			bad = 1;
		fp = NULL;
		/* same bytes as lm_save_checkpoint: the Adam section goes right after the weights */
		if (!bad && anni_ckpt_write_adam(tmp, 1, k->epoch, k->step, k->t, n, m, v) != ANNI_OK)
			bad = 1;
	} else if (!bad)
		bad |= wr32(fp, 0);	/* lm_save: "no adam section" */
	if (fp && fclose(fp) != 0)
		bad = 1;
	if (bad || rename(tmp, path) != 0) {
		remove(tmp);
		return ANNI_E_ARG;
	}
	return ANNI_OK;
}
