/* wr_b200_host.h — shared by the host objects that replace the reference's
 * session.c / batch.c and wrap its engine entry points. */
#ifndef WR_B200_HOST_H
#define WR_B200_HOST_H

#include "wr_cuda.h"

/* The process's device context (owned by the engine gate, wr_b200_engine.c).
 * NULL and a negative *rc_out when no B200 is bound. */
wr_cuda_ctx *wr_b200_cuda_ctx(int *rc_out);

#endif
