/* C acceptance program for the tensor_ash.h ABI, written for this repository.
 * It walks the same sequence a C embedder of the reference library would
 * (the reference ships examples/c_smoke.c for that purpose): context and
 * executor creation, tensor upload, a plain GEMM with the known answer
 * {58, 64, 139, 154}, a fused bias+SiLU op, prepared run/submit/wait, an
 * f16-weight GEMM, rms_norm, prefix softmax, a strided transpose and the
 * rejection of an in-place strided copy.  Exit code 0 means every check held. */
#include <math.h>
#include <stdio.h>
#include <string.h>

#include "tensor_ash.h"

static int failures = 0;
#define EXPECT(cond, ...)                  \
  do {                                     \
    if (!(cond)) {                         \
      fprintf(stderr, "FAIL: " __VA_ARGS__); \
      fprintf(stderr, " [%s]\n", ta_last_error()); \
      ++failures;                          \
    }                                      \
  } while (0)

static int near(float a, float b, float tol) { return fabsf(a - b) <= tol; }

int main(void) {
  ta_context *ctx = ta_context_create(0, "auto");
  if (!ctx) { fprintf(stderr, "context: %s\n", ta_last_error()); return 1; }
  ta_executor *ex = ta_executor_create(ctx, 2, 16, "auto");
  if (!ex) { fprintf(stderr, "executor: %s\n", ta_last_error()); return 1; }
  EXPECT(strcmp(ta_version(), "2.0.0") == 0, "version");
  EXPECT(ta_context_supports_f16(ctx) == 1 && ta_context_supports_bda(ctx) == 1, "capabilities");

  const uint32_t s23[2] = {2, 3}, s32[2] = {3, 2}, s22[2] = {2, 2}, s2[1] = {2}, s3[1] = {3};
  ta_tensor *a = ta_tensor_create(ctx, s23, 2), *b = ta_tensor_create(ctx, s32, 2);
  ta_tensor *c = ta_tensor_create_on_executor(ex, s22, 2);
  EXPECT(a && b && c, "tensor create");
  EXPECT(ta_tensor_len(a) == 6 && ta_tensor_size_bytes(a) == 32, "len/size (24 B rounds up to 32)");
  const float ha[6] = {1, 2, 3, 4, 5, 6}, hb[6] = {7, 8, 9, 10, 11, 12};
  float hc[4] = {0};
  EXPECT(ta_upload(ex, a, ha, 6) == 0 && ta_upload(ex, b, hb, 6) == 0, "upload");

  ta_run_stats st;
  memset(&st, 0, sizeof st);
  EXPECT(ta_matmul(ex, a, b, c, 1.0f, 0, &st) == 0, "ta_matmul");
  EXPECT(ta_download(ex, c, hc, 4) == 0, "download");
  const float want[4] = {58, 64, 139, 154};
  for (int i = 0; i < 4; ++i) EXPECT(near(hc[i], want[i], 1e-4f), "matmul c[%d]=%f", i, hc[i]);
  EXPECT(st.n_calls == 1 && st.total_flops == 24 && st.has_gpu_time == 1, "stats");

  ta_dispatch_info info;
  memset(&info, 0, sizeof info);
  EXPECT(ta_dispatch_info_for(ex, 1, 2, 2, 3, 0, &info) == 0 && info.kernel && info.tile[0] > 0, "dispatch info");

  /* fused bias + SiLU: c00 = 58 - 58.5 = -0.5 -> silu(-0.5) */
  ta_tensor *bias = ta_tensor_create(ctx, s2, 1);
  const float hbias[2] = {-58.5f, 0.0f};
  EXPECT(ta_upload(ex, bias, hbias, 2) == 0, "upload bias");
  ta_matmul_op op;
  memset(&op, 0, sizeof op);
  op.call.a = a; op.call.b = b; op.call.c = c; op.call.alpha = 1.0f;
  op.epilogue.bias = bias; op.epilogue.activation = TA_ACTIVATION_SILU;
  EXPECT(ta_run_ops(ex, &op, 1, &st) == 0, "ta_run_ops");
  EXPECT(ta_download(ex, c, hc, 4) == 0, "download 2");
  EXPECT(near(hc[0], -0.5f / (1.0f + expf(0.5f)), 1e-5f) && near(hc[1], 64.0f, 1e-3f), "bias+silu %f %f", hc[0], hc[1]);

  /* invalid enum and dangling d are rejected */
  op.epilogue.activation = 9;
  EXPECT(ta_run_ops(ex, &op, 1, NULL) == -1 && strstr(ta_last_error(), "activation 9 is invalid"), "bad activation");
  op.epilogue.activation = 0; op.epilogue.d = c;
  EXPECT(ta_run_ops(ex, &op, 1, NULL) == -1 && strstr(ta_last_error(), "binary_kind is 0"), "d without binary");

  /* prepared replay */
  ta_matmul_op plain;
  memset(&plain, 0, sizeof plain);
  plain.call.a = a; plain.call.b = b; plain.call.c = c; plain.call.alpha = 1.0f;
  ta_prepared *prep = ta_prepared_create(ex, &plain, 1, 0);
  EXPECT(prep != NULL, "prepared create");
  if (prep) {
    EXPECT(ta_prepared_wait(prep, &st) == -1, "wait without submit");
    EXPECT(ta_prepared_run(prep, &st) == 0 && ta_prepared_run(prep, &st) == 0, "prepared run x2");
    EXPECT(ta_prepared_submit(prep) == 0, "prepared submit");
    EXPECT(ta_prepared_submit(prep) == -1, "double submit");
    EXPECT(ta_prepared_wait(prep, &st) == 0, "prepared wait");
    EXPECT(ta_download(ex, c, hc, 4) == 0, "download 3");
    for (int i = 0; i < 4; ++i) EXPECT(near(hc[i], want[i], 1e-4f), "prepared c[%d]=%f", i, hc[i]);
    ta_prepared_destroy(prep);
  }

  /* f16 weight storage */
  ta_tensor *b16 = ta_tensor_create_f16(ctx, s32, 2);
  EXPECT(b16 && ta_tensor_is_f16(b16) == 1 && ta_tensor_is_f16(b) == 0, "f16 tensor");
  EXPECT(ta_upload(ex, b16, hb, 6) == 0 && ta_matmul(ex, a, b16, c, 1.0f, 0, &st) == 0, "f16 matmul");
  EXPECT(ta_download(ex, c, hc, 4) == 0 && near(hc[0], 58.0f, 1e-3f), "f16 result %f", hc[0]);

  /* rms_norm, prefix softmax, transpose */
  ta_tensor *w = ta_tensor_create(ctx, s3, 1), *o23 = ta_tensor_create(ctx, s23, 2), *o32 = ta_tensor_create(ctx, s32, 2);
  const float hw[3] = {1.0f, 0.5f, 2.0f};
  float ho[6];
  EXPECT(ta_upload(ex, w, hw, 3) == 0 && ta_rms_norm(ex, a, w, o23, 1e-5f, &st) == 0, "rms_norm");
  EXPECT(ta_download(ex, o23, ho, 6) == 0, "download rms");
  for (int r = 0; r < 2; ++r) {
    float ss = 0;
    for (int j = 0; j < 3; ++j) ss += ha[3 * r + j] * ha[3 * r + j];
    const float inv = 1.0f / sqrtf(ss / 3.0f + 1e-5f);
    for (int j = 0; j < 3; ++j) EXPECT(near(ho[3 * r + j], ha[3 * r + j] * hw[j] * inv, 1e-4f), "rms[%d,%d]", r, j);
  }
  EXPECT(ta_softmax_rows(ex, a, o23, 1.0f, TA_SOFTMAX_MASK_PREFIX, 2, 0, &st) == 0 && ta_download(ex, o23, ho, 6) == 0, "softmax");
  for (int r = 0; r < 2; ++r) {
    const float e0 = expf(ha[3 * r] - ha[3 * r + 1]), e1 = 1.0f;
    EXPECT(near(ho[3 * r], e0 / (e0 + e1), 1e-5f) && near(ho[3 * r + 1], e1 / (e0 + e1), 1e-5f) && ho[3 * r + 2] == 0.0f, "softmax row %d", r);
  }
  ta_copy_desc tr;
  memset(&tr, 0, sizeof tr);
  tr.extent[0] = 3; tr.extent[1] = 2; tr.extent[2] = 1;
  tr.src_strides[0] = 1; tr.src_strides[1] = 3; tr.dst_strides[0] = 2; tr.dst_strides[1] = 1;
  EXPECT(ta_copy_strided(ex, a, o32, &tr, &st) == 0 && ta_download(ex, o32, ho, 6) == 0, "copy_strided");
  const float wt[6] = {1, 4, 2, 5, 3, 6};
  for (int i = 0; i < 6; ++i) EXPECT(ho[i] == wt[i], "transpose[%d]=%f", i, ho[i]);
  EXPECT(ta_copy_strided(ex, a, a, &tr, NULL) == -1, "in-place copy must be rejected");

  ta_tensor_destroy(o32); ta_tensor_destroy(o23); ta_tensor_destroy(w); ta_tensor_destroy(b16);
  ta_tensor_destroy(bias); ta_tensor_destroy(c); ta_tensor_destroy(b); ta_tensor_destroy(a);
  ta_executor_destroy(ex);
  ta_context_destroy(ctx);
  if (failures) { fprintf(stderr, "%d check(s) failed\n", failures); return 2; }
  printf("tensor-ash C ABI smoke OK\n");
  return 0;
}
