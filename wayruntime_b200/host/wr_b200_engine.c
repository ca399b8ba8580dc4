/*
 * wr_b200_engine.c — the B200 gate of wr_engine_create, and the owner of the
 * process's device context.
 *
 * The reference creates its engine after one host probe (little-endian,
 * src/core/engine.c:119-167, probe at :130) and promises "errors, never
 * guesses": an unsupported host gets WR_ERR_UNSUPPORTED, not a degraded path
 * (include/wayruntime/wayruntime.h:181-185).  With attention on the GPU the
 * same promise needs one more probe: no compute-capability-10.x device bound
 * to the process -> WR_ERR_UNSUPPORTED from wr_engine_create itself, with one
 * log line, and no CPU attention anywhere behind it.
 *
 * The reference's engine.c is compiled unmodified, with its two entry points
 * renamed on the compiler's command line (-Dwr_engine_create=
 * wri_ref_engine_create, -Dwr_engine_destroy=wri_ref_engine_destroy); this
 * file exports the public names, probes, creates the device context, and
 * calls through.  The context lives as long as the engine.
 *
 * Environment: WR_CUDA_DEVICE selects the device (default 0).
 */
#include <stdlib.h>

#include "core/internal.h"
#include "wr_b200_host.h"
#include "wr_cuda.h"

wr_status wri_ref_engine_create(const wr_engine_config *cfg, wr_engine **out);
void      wri_ref_engine_destroy(wr_engine *e);

static wr_cuda_ctx *g_cuda;            /* one per process, like the engine */
static volatile int g_cuda_guard;      /* creation / release are rare: a flag is enough */

static void guard_lock(void)   { while (__atomic_exchange_n(&g_cuda_guard, 1, __ATOMIC_ACQUIRE)) { } }
static void guard_unlock(void) { __atomic_store_n(&g_cuda_guard, 0, __ATOMIC_RELEASE); }

static int cuda_device_index(void)
{
    const char *dev = getenv("WR_CUDA_DEVICE");
    return dev ? atoi(dev) : 0;
}

/* The process's device context; created on first use when no engine made it
 * (the self-tests run without an engine).  NULL + *rc_out < 0 without a B200. */
wr_cuda_ctx *wr_b200_cuda_ctx(int *rc_out)
{
    guard_lock();
    int rc = 0;
    if (!g_cuda) {
        rc = wr_cuda_ctx_create(cuda_device_index(), &g_cuda);
        if (rc == 0) {
            rc = wr_cuda_ctx_set_attn_max_seq(g_cuda, WR_ATTN_MAX_SEQ);
            if (rc != 0) {
                wr_cuda_ctx_destroy(g_cuda);
                g_cuda = NULL;
            }
        }
    }
    wr_cuda_ctx *c = g_cuda;
    guard_unlock();
    if (rc_out) *rc_out = rc;
    return c;
}

static void cuda_release(void)
{
    guard_lock();
    wr_cuda_ctx *c = g_cuda;
    g_cuda = NULL;
    guard_unlock();
    if (c) wr_cuda_ctx_destroy(c);
}

static void gate_log(const wr_engine_config *cfg, const char *line)
{
    /* no engine exists yet, so the caller's sink is reached through its config */
    if (cfg && cfg->log_fn) cfg->log_fn(0, line, cfg->log_user);
    else wri_log_msg(0, "%s", line);
}

wr_status wr_engine_create(const wr_engine_config *cfg, wr_engine **out)
{
    if (out == NULL) return WR_ERR_INVAL;
    *out = NULL;
    if (wr_cuda_device_check(cuda_device_index()) != 0) {
        gate_log(cfg, "engine_create: no compute-capability-10.x (B200) device is bound to this "
                      "process; attention has no CPU path here (WR_ERR_UNSUPPORTED)");
        return WR_ERR_UNSUPPORTED;
    }
    if (wri_g_engine == NULL) {                  /* (a second engine is refused by the reference below) */
        int rc = 0;
        if (!wr_b200_cuda_ctx(&rc)) {
            gate_log(cfg, "engine_create: the device context could not be created");
            return (rc == WR_ERR_NOMEM) ? WR_ERR_NOMEM : (rc < 0 ? (wr_status)rc : WR_ERR_INTERNAL);
        }
    }
    wr_status st = wri_ref_engine_create(cfg, out);
    if (st != WR_OK && wri_g_engine == NULL) cuda_release();
    return st;
}

void wr_engine_destroy(wr_engine *e)
{
    wri_ref_engine_destroy(e);                   /* refuses while models are live */
    if (wri_g_engine == NULL) cuda_release();
}
