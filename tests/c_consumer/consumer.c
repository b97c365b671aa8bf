/* A plain C11 consumer of include/fln_b200.h: what a maintainer of the reference would write
 * in place of its pybind launchers (csrc/bindings.cpp:3-17 of the reference declares its
 * launchers as extern "C" functions that take at::Tensor by value, which C cannot call; this
 * header can be).  Only host-side entry points are called, so it runs without a GPU.
 * Built and run by tests/test_c_consumer.py:  gcc -std=c11 -Wall -Werror -pedantic. */
#include <stdio.h>
#include <string.h>

#include "fln_b200.h"

static int failures = 0;
#define EXPECT(cond)                                             \
  do {                                                           \
    if (!(cond)) {                                               \
      printf("FAILED line %d: %s\n", __LINE__, #cond);           \
      ++failures;                                                \
    }                                                            \
  } while (0)

int main(void) {
  /* version attributes */
  EXPECT(strcmp(fln_version(), "1.0.0") == 0);
  EXPECT(fln_cuda_runtime_version() >= 12000);
  EXPECT(strcmp(fln_status_string(FLN_OK), "ok") == 0);
  EXPECT(strlen(fln_status_string(FLN_ERR_STATIC_SCRATCH)) > 0);

  /* closed-form memory estimate: 2MNe + 2M*4 + MNe + 2Ne + M*32*4 */
  const int m = 32, n = 4096;
  const int64_t want = 2LL * m * n * 4 + 2LL * m * 4 + 1LL * m * n * 4 + 2LL * n * 4 + 1LL * m * 32 * 4;
  EXPECT(fln_get_memory_usage(m, n, 0) == want);

  char hints[1024];
  const int len = fln_get_performance_hints(4, 1000, hints, sizeof hints);
  EXPECT(len > 0 && (size_t)len == strlen(hints));
  EXPECT(strstr(hints, "not divisible by 32") != NULL);

  /* launch planning is pure host code */
  fln_launch_info info;
  EXPECT(fln_describe_launch(0, 16384, 8192, FLN_BF16, 1, &info) == FLN_OK);
  EXPECT(info.pipelined == 1 && info.vec_elems == 8 && info.stages >= 2);
  EXPECT(fln_describe_launch(1, 32, 4096, FLN_F32, 1, &info) == FLN_OK);
  EXPECT(info.pipelined == 0);
  EXPECT(fln_planner_selftest() == 0);
  EXPECT(fln_backward_workspace_bytes(0, 8, FLN_F32) == 0);
  EXPECT(fln_backward_workspace_bytes(16384, 8192, FLN_BF16) <= FLN_STATIC_SCRATCH_BYTES);

  /* argument errors come back as status codes before anything touches a device */
  EXPECT(fln_layernorm_forward(NULL, NULL, NULL, NULL, NULL, NULL, 4, 8, 7, 1e-5f, NULL) == FLN_ERR_DTYPE);
  EXPECT(fln_layernorm_forward(NULL, NULL, NULL, NULL, NULL, NULL, 4, 0, FLN_F32, 1e-5f, NULL) == FLN_ERR_SHAPE);
  EXPECT(fln_layernorm_forward(NULL, NULL, NULL, NULL, NULL, NULL, 4, 8, FLN_F32, 1e-5f, NULL) == FLN_ERR_NULL);
  EXPECT(fln_layernorm_gelu_forward(NULL, NULL, NULL, NULL, 4, 8, FLN_F32, 1e-5f, FLN_ACT_NONE, NULL) == FLN_ERR_ARG);
  EXPECT(fln_norm_backward(FLN_LAYERNORM, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, 0, 4, 8,
                           9, NULL) == FLN_ERR_DTYPE);
  EXPECT(fln_layernorm_backward_static(NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL, -1, 8, FLN_F32, NULL) ==
         FLN_ERR_SHAPE);
  EXPECT(fln_sum_rows_f32(NULL, 0, 8, NULL, NULL, FLN_F32, NULL) == FLN_ERR_SHAPE);

  /* tuning hooks are plain setters */
  fln_set_plan_override(0, 0);
  fln_set_path_override(0);
  fln_set_stage_override(0);
  fln_set_sm_reserve(0);
  fln_set_static_scratch_limit(0);
  EXPECT(fln_set_wait_limit_ns(0) == FLN_OK);

  if (failures == 0) printf("c consumer ok: %s, cuda runtime %d\n", fln_version(), fln_cuda_runtime_version());
  return failures;
}
