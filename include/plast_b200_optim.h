/*
 * plast_b200_optim.h — optimiser steps of the plast runtime on sm_100a: one multi-tensor launch
 * updates every parameter of a step (bandwidth-bound elementwise work, like the rest of this
 * library).
 *
 * Replaces src/optimizers/cuda/{sgd,adam,adamw}.cu. The reference's sgd_step_cuda launches one
 * scalar kernel per parameter (sgd.cu:11-32); its adam_step_cuda and adamw_step_cuda are empty
 * functions (adam.cu:17-18, adamw.cu:20-21), so the arithmetic contract is the CPU path:
 * src/optimizers/cpu/sgd.c:11-32, adam.c:22-72, adamw.c:21-74. Parameters, gradients and moments
 * are treated as flat float arrays of numel(param) elements, as the CPU loops do; parameters
 * that are NULL or have no grad are skipped.
 *
 * SGD, Adam and AdamW restate include/optimizers/{sgd,adam,adamw}.h; define
 * PLAST_B200_USE_REFERENCE_TYPES to compile against the reference's own headers instead.
 */
#ifndef PLAST_B200_OPTIM_H
#define PLAST_B200_OPTIM_H

#include "plast_b200.h"

#ifdef PLAST_B200_USE_REFERENCE_TYPES
#include "optimizers/adam.h"
#include "optimizers/adamw.h"
#include "optimizers/sgd.h"
#else

struct Arena;

/* include/optimizers/sgd.h:5-7 */
typedef struct {
  float lr;
} SGD;

/* include/optimizers/adam.h:5-15 — 56 bytes: lr@0 beta1@4 beta2@8 epsilon@12 t@16 m@24 v@32 */
typedef struct {
  float lr;
  float beta1;
  float beta2;
  float epsilon;
  int t;
  Tensor **m;
  Tensor **v;
  struct Arena *data_arena;
  struct Arena *optimizer_arena;
} Adam;

/* include/optimizers/adamw.h:5-16 — 56 bytes: ... weight_decay@16 t@20 m@24 v@32 */
typedef struct {
  float lr;
  float beta1;
  float beta2;
  float epsilon;
  float weight_decay;
  int t;
  Tensor **m;
  Tensor **v;
  struct Arena *data_arena;
  struct Arena *optimizer_arena;
} AdamW;

#endif /* PLAST_B200_USE_REFERENCE_TYPES */

#ifdef __cplusplus
extern "C" {
#endif

/* data[j] -= lr * grad[j] (src/optimizers/cpu/sgd.c:28-30); product and difference each
 * rounded to fp32. */
void sgd_step_cuda(SGD *optimizer, Tensor **parameters, int num_parameters);

/* optimizer->t is incremented first; on the first step the moment tensors are created, zeroed,
 * and stored in optimizer->m / optimizer->v (the CPU path takes them from the optimizer's
 * arenas, adam.c:30-46; here the library owns them: one device allocation for all moments and
 * host Tensor structs, freed by plast_b200_adam_state_release). Then, with
 *   lr_t = lr * sqrt(1 - beta2^t) / (1 - beta1^t)   (computed on the host exactly as adam.c:48-49)
 * every element does, each operation rounded to fp32 (adam.c:62-66):
 *   m = beta1 * m + (1 - beta1) * g;  v = beta2 * v + (1 - beta2) * g * g;
 *   data -= lr_t * m / (sqrtf(v) + epsilon)
 * AdamW first applies data -= lr * weight_decay * data (adamw.c:65-66). */
void adam_step_cuda(Adam *optimizer, Tensor **parameters, int num_parameters);
void adamw_step_cuda(AdamW *optimizer, Tensor **parameters, int num_parameters);

/* Frees moments created by adam_step_cuda / adamw_step_cuda (pass optimizer->m, optimizer->v)
 * and leaves nothing behind; unknown pointers are ignored. No reference counterpart: the
 * reference releases its arenas as a whole. */
void plast_b200_adam_state_release(Tensor **m, Tensor **v);

#ifdef __cplusplus
}
#endif

#endif /* PLAST_B200_OPTIM_H */
