// Loss helpers with the call signatures of dl-cuda's src/loss.cuh (:7-12,
// :146-221): per-sample errors and gradients for squared, absolute, binary and
// categorical cross-entropy losses, and the cross entropy against integer
// targets that the char-LM example trains with.  All of them are one call into
// the kernel library.
#pragma once

#include "sequential.cuh"

enum LossType { SQUARED_ERROR, ABSOLUTE_ERROR, BINARY_CROSS_ENTROPY, CATEGORICAL_CROSS_ENTROPY };

static const int LOSS_ELEMENTS_PER_THREAD = 2;

inline int dlb_loss_kind(LossType loss_type) {
  switch (loss_type) {
  case SQUARED_ERROR: return DLB_LOSS_SQUARED;
  case ABSOLUTE_ERROR: return DLB_LOSS_ABSOLUTE;
  case BINARY_CROSS_ENTROPY: return DLB_LOSS_BCE;
  case CATEGORICAL_CROSS_ENTROPY: return DLB_LOSS_CCE;
  }
  return -1;
}

// error[n] from targets y and predictions y_pred (both [n], or [n, classes] for
// the categorical loss).  The launch shape arguments are accepted for source
// compatibility; the library sizes its own grid.
inline void computeLoss(float *y, float *y_pred, float *error, int n, int classes, LossType loss_type,
                        dim3 /*blocks*/, dim3 /*threads*/) {
  const int kind = dlb_loss_kind(loss_type);
  if (kind < 0) {
    printf("Invalid loss type\n");
    return;
  }
  DLB_CHECK(dlb_loss_fwd(kind, y, y_pred, error, n, classes, nullptr));
}

// d(mean loss)/d(y_pred), same shape as y_pred.
inline void computeLossBackward(float *y, float *y_pred, float *grad, int n, int classes,
                                LossType loss_type) {
  const int kind = dlb_loss_kind(loss_type);
  if (kind < 0) {
    printf("Unsupported loss type for backward\n");
    return;
  }
  DLB_CHECK(dlb_loss_bwd(kind, y, y_pred, grad, n, classes, nullptr));
}

inline void computeCategoricalCrossEntropyFromIds(const int *target_ids, const float *y_pred, float *error,
                                                  int n, int classes, float epsilon = 1e-10f) {
  DLB_CHECK(dlb_ce_from_ids_fwd(target_ids, y_pred, error, n, classes, epsilon, nullptr));
}

inline void computeCategoricalCrossEntropyBackwardFromIds(const int *target_ids, const float *y_pred,
                                                          float *grad, int n, int classes,
                                                          float epsilon = 1e-10f) {
  DLB_CHECK(dlb_ce_from_ids_bwd(target_ids, y_pred, grad, n, classes, epsilon, nullptr));
}
