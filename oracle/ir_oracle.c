/*
 * CPU oracle: a plain-C interpreter of the reference's HLIR (`enum IRCmds`,
 * src/core/ir.rs:8-105).  TEST INFRASTRUCTURE ONLY: it is the checker the CUDA
 * backend is compared against and the timed CPU baseline; nothing in the product
 * library links or calls it.
 *
 * Pinning: the interpreter is run against every known-answer vector the reference's
 * own tests carry (src/tests/{ct,ctrl,eq,evryt,grd,nn,norm}.rs) and against PyTorch
 * CPU on the same programs the reference's src/pytest scripts use; see tests/.
 *
 * What each part restates:
 *   per-element arithmetic   src/devices/opencl/kernels/unary.rs:3-17 (exp2, log2, sin,
 *                            1.0/x, sqrt(fabs(x)), ==0 / >0 / <0 -> 1.0/0.0) and
 *                            binary.rs:3-14 (+, *)
 *   row sum                  src/devices/opencl/kernels/reduce.rs:4-11,40-55 (the
 *                            mathematically specified sum over the last axis, y ascending)
 *   dot product              src/devices/opencl/kernels/dotprod.rs:28-46
 *                            (`value += a*b`, k ascending, fp32)
 *   alias tracking           src/kernel/trackers/kernel.rs:76-232 (View / Index / Permute /
 *                            Broadcast never move data; Concat is a two-way select)
 *   index mapping            src/kernel/helper/shape.rs:13-76 and
 *                            src/kernel/indexing/matrix.rs:11-60 (reverse application of
 *                            the data commands; concat picks `b` when idx[dim] > idx_end-1)
 *   control flow             src/devices/opencl/device.rs:107-146 (If tests == 1.0, While
 *                            tests != 0.0, EX unwinds everything)
 *   read-back                src/devices/opencl/device.rs:82-102 (only ids in the dep list)
 *
 * Deliberate, documented choices where the reference is broken or silent:
 *   - Index re-inserts the removed axis and Permute maps sink axis i to source axis p[i]
 *     (the shape rule of src/kernel/trackers/shape.rs), also for non-involutive p.
 *   - An op-assign whose target id is an alias (or a constant) rebinds the id to a fresh
 *     buffer holding the result; the reference has no buffer for such ids.
 *   - A dep-list id that is an alias is materialised on read-back instead of panicking.
 *   - Every op computes into a fresh array and then replaces the target (value semantics),
 *     so reads through permuted aliases of the target never observe partial updates.
 *
 * Transcendentals use glibc's exp2f/log2f/sinf/sqrtf and IEEE division; build with
 * -ffp-contract=off so a*b+c is two roundings, as in the reference's non-fused kernels.
 */
#define _GNU_SOURCE
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define MAXD 8

enum { K_UNDEF = 0, K_BUF, K_CONST, K_ALIAS, K_CONCAT };
enum { A_VIEW = 0, A_INDEX, A_PERMUTE, A_BROADCAST };

typedef struct {
    int kind;
    int nd;
    uint64_t dims[MAXD];
    float *data; /* K_BUF */
    int borrowed; /* K_BUF whose storage belongs to the caller */
    float cval;  /* K_CONST */
    /* K_ALIAS */
    int parent, acmd, adim;
    uint64_t aindex;
    int perm[MAXD];
    int src_nd;
    uint64_t src_dims[MAXD];
    /* K_CONCAT */
    int ca, cb, cdim;
    uint64_t idx_end;
} Var;

typedef struct Cmd Cmd;
typedef struct { Cmd *cmds; uint32_t n; } Proc;
struct Cmd {
    uint8_t op;
    uint32_t a, b, res;
    int nd;
    uint64_t dims[MAXD];
    uint32_t perm[MAXD];
    uint64_t index, count;
    uint32_t dim;
    float cval;
    const float *payload;
    uint8_t payload_kind;
    Proc block;         /* While */
    uint32_t ncond;     /* If */
    uint32_t *cond_ids;
    Proc *cond_blocks;
    int has_else;
    Proc else_block;
    uint32_t pos;       /* textual position (top-level index of the enclosing top-level command) */
};

typedef void (*allreduce_fn)(float *data, uint64_t n, void *user);

typedef struct {
    uint32_t n_ids;
    char **names;
    Var *vars;
    uint32_t n_dep;
    uint32_t *dep;
    uint8_t *is_dep;
    Proc main;
    uint32_t *last_use;
    int stop;
    char err[512];
    /* results */
    uint32_t n_res;
    char **res_names;
    float **res_data;
    uint64_t (*res_dims)[MAXD];
    int *res_nd;
    allreduce_fn allreduce;
    void *allreduce_user;
    int f64_acc;
    uint64_t cmds_executed;
} Oracle;

/* ------------------------------------------------------------------ parsing */
typedef struct { const uint8_t *p, *base, *end; int bad; } Rd;
static uint8_t r8(Rd *r) { if (r->p + 1 > r->end) { r->bad = 1; return 0; } return *r->p++; }
static uint16_t r16(Rd *r) { uint16_t v = 0; if (r->p + 2 > r->end) { r->bad = 1; return 0; } memcpy(&v, r->p, 2); r->p += 2; return v; }
static uint32_t r32(Rd *r) { uint32_t v = 0; if (r->p + 4 > r->end) { r->bad = 1; return 0; } memcpy(&v, r->p, 4); r->p += 4; return v; }
static uint64_t r64(Rd *r) { uint64_t v = 0; if (r->p + 8 > r->end) { r->bad = 1; return 0; } memcpy(&v, r->p, 8); r->p += 8; return v; }
static float rf32(Rd *r) { float v = 0; if (r->p + 4 > r->end) { r->bad = 1; return 0; } memcpy(&v, r->p, 4); r->p += 4; return v; }

static int parse_proc(Oracle *o, Rd *r, Proc *out, int depth);

static void rdims(Rd *r, Cmd *c) {
    c->nd = r8(r);
    if (c->nd > MAXD) { r->bad = 1; c->nd = 0; return; }
    for (int i = 0; i < c->nd; i++) c->dims[i] = r64(r);
}

static int parse_cmd(Oracle *o, Rd *r, Cmd *c, int depth) {
    memset(c, 0, sizeof(*c));
    c->op = r8(r);
    switch (c->op) {
    case 1:
        c->res = r32(r); rdims(r, c); c->payload_kind = r8(r);
        { uint64_t v = r64(r); c->count = r64(r);
          if (c->payload_kind == 0) c->payload = (const float *)(r->base + v);
          else if (c->payload_kind == 1) c->payload = (const float *)(uintptr_t)v;
          else { snprintf(o->err, sizeof o->err, "oracle: device-resident payload unsupported"); return -1; } }
        break;
    case 2: c->res = r32(r); c->cval = rf32(r); rdims(r, c); break;
    case 3: case 4: case 11: case 29: c->a = r32(r); c->b = r32(r); c->res = r32(r); break;
    case 5: case 6: c->a = r32(r); c->b = r32(r); c->res = c->a; break;
    case 7: case 8: case 9: case 10: case 17: case 18: case 19: case 20: case 21: case 22: case 28:
        c->a = r32(r); c->res = r32(r); break;
    case 12: c->a = r32(r); c->res = r32(r); rdims(r, c); break;
    case 13: c->a = r32(r); c->res = r32(r); c->index = r64(r); c->dim = r32(r); break;
    case 14: c->a = r32(r); c->b = r32(r); c->res = r32(r); c->dim = r32(r); break;
    case 15: c->a = r32(r); c->res = r32(r); c->nd = r8(r);
        if (c->nd > MAXD) { r->bad = 1; return -1; }
        for (int i = 0; i < c->nd; i++) c->perm[i] = r32(r);
        break;
    case 16: c->a = r32(r); c->res = r32(r); c->dim = r32(r); c->count = r64(r); break;
    case 23: c->a = r32(r); if (parse_proc(o, r, &c->block, depth + 1)) return -1; break;
    case 24:
        c->ncond = r32(r);
        if (c->ncond > 1u << 20) { r->bad = 1; return -1; }
        c->cond_ids = calloc(c->ncond ? c->ncond : 1, sizeof(uint32_t));
        c->cond_blocks = calloc(c->ncond ? c->ncond : 1, sizeof(Proc));
        for (uint32_t i = 0; i < c->ncond; i++) {
            c->cond_ids[i] = r32(r);
            if (parse_proc(o, r, &c->cond_blocks[i], depth + 1)) return -1;
        }
        c->has_else = r8(r);
        if (c->has_else && parse_proc(o, r, &c->else_block, depth + 1)) return -1;
        break;
    case 25: break;
    case 26: { uint16_t n = r16(r); if (r->p + n > r->end) r->bad = 1; else r->p += n; } break;
    case 27: c->a = r32(r); c->res = c->a; break;
    default:
        snprintf(o->err, sizeof o->err, "oracle: unknown opcode %u", c->op);
        return -1;
    }
    if (r->bad) { snprintf(o->err, sizeof o->err, "oracle: truncated blob"); return -1; }
    if (c->a >= o->n_ids || c->b >= o->n_ids || c->res >= o->n_ids) {
        snprintf(o->err, sizeof o->err, "oracle: id index out of range"); return -1;
    }
    return 0;
}

static int parse_proc(Oracle *o, Rd *r, Proc *out, int depth) {
    if (depth > 64) { snprintf(o->err, sizeof o->err, "oracle: nesting too deep"); return -1; }
    out->n = r32(r);
    if (r->bad || out->n > (1u << 28)) { snprintf(o->err, sizeof o->err, "oracle: bad procedure"); return -1; }
    out->cmds = calloc(out->n ? out->n : 1, sizeof(Cmd));
    for (uint32_t i = 0; i < out->n; i++)
        if (parse_cmd(o, r, &out->cmds[i], depth)) return -1;
    return 0;
}

static void free_proc(Proc *p) {
    for (uint32_t i = 0; i < p->n; i++) {
        Cmd *c = &p->cmds[i];
        if (c->op == 23) free_proc(&c->block);
        if (c->op == 24) {
            for (uint32_t k = 0; k < c->ncond; k++) free_proc(&c->cond_blocks[k]);
            free(c->cond_ids); free(c->cond_blocks);
            if (c->has_else) free_proc(&c->else_block);
        }
    }
    free(p->cmds);
    p->cmds = NULL; p->n = 0;
}

/* ------------------------------------------------------------------ liveness (memory only) */
static void mark_use(Oracle *o, uint32_t id, uint32_t pos) { if (o->last_use[id] < pos) o->last_use[id] = pos; }

static void scan_uses(Oracle *o, Proc *p, int top, uint32_t outer_pos) {
    for (uint32_t i = 0; i < p->n; i++) {
        Cmd *c = &p->cmds[i];
        uint32_t pos = top ? i : outer_pos;
        c->pos = pos;
        switch (c->op) {
        case 3: case 4: case 11: case 14: case 29: mark_use(o, c->a, pos); mark_use(o, c->b, pos); break;
        case 5: case 6: mark_use(o, c->a, pos); mark_use(o, c->b, pos); break;
        case 7: case 8: case 9: case 10: case 12: case 13: case 15: case 16: case 17:
        case 18: case 19: case 20: case 21: case 22: case 27: case 28:
            mark_use(o, c->a, pos); break;
        case 23: mark_use(o, c->a, pos); scan_uses(o, &c->block, 0, pos); break;
        case 24:
            for (uint32_t k = 0; k < c->ncond; k++) { mark_use(o, c->cond_ids[k], pos); scan_uses(o, &c->cond_blocks[k], 0, pos); }
            if (c->has_else) scan_uses(o, &c->else_block, 0, pos);
            break;
        default: break;
        }
    }
}

/* an alias keeps its parents alive: propagate in reverse textual order */
static void propagate_alias(Oracle *o, Proc *p) {
    for (uint32_t ii = p->n; ii-- > 0;) {
        Cmd *c = &p->cmds[ii];
        if (c->op == 23) propagate_alias(o, &c->block);
        else if (c->op == 24) {
            if (c->has_else) propagate_alias(o, &c->else_block);
            for (uint32_t k = c->ncond; k-- > 0;) propagate_alias(o, &c->cond_blocks[k]);
        } else if (c->op == 12 || c->op == 13 || c->op == 15 || c->op == 16) {
            mark_use(o, c->a, o->last_use[c->res]);
        } else if (c->op == 14) {
            mark_use(o, c->a, o->last_use[c->res]); mark_use(o, c->b, o->last_use[c->res]);
        }
    }
}

/* ------------------------------------------------------------------ buffer pool
 * Large arrays come and go with every command; recycling them avoids the page-fault cost of fresh
 * mappings (this only affects speed of the CPU baseline, never values). */
#define POOL_SLOTS 96
static struct { float *p; size_t cap; } g_pool[POOL_SLOTS];
static size_t g_pool_bytes = 0;

static float *pool_alloc(size_t n) {
    if (n == 0) n = 1;
    int best = -1;
#pragma omp critical(adb_pool)
    {
        for (int i = 0; i < POOL_SLOTS; i++)
            if (g_pool[i].p && g_pool[i].cap >= n && g_pool[i].cap <= 2 * n + 1024 && (best < 0 || g_pool[i].cap < g_pool[best].cap)) best = i;
    }
    if (best >= 0) {
        float *p = g_pool[best].p;
        g_pool_bytes -= g_pool[best].cap * sizeof(float);
        g_pool[best].p = NULL;
        /* remember the capacity in a header word in front of the array */
        return p;
    }
    size_t *raw = malloc(sizeof(float) * n + 64);
    raw[0] = n;
    return (float *)((char *)raw + 64);
}

static void pool_free(float *p) {
    if (!p) return;
    size_t *raw = (size_t *)((char *)p - 64);
    size_t cap = raw[0];
    if (cap >= (1u << 16) && g_pool_bytes + cap * sizeof(float) < ((size_t)12 << 30)) {
        for (int i = 0; i < POOL_SLOTS; i++)
            if (!g_pool[i].p) {
                g_pool[i].p = p;
                g_pool[i].cap = cap;
                g_pool_bytes += cap * sizeof(float);
                return;
            }
    }
    free(raw);
}

/* ------------------------------------------------------------------ helpers */
static uint64_t numel(const Var *v) { uint64_t n = 1; for (int i = 0; i < v->nd; i++) n *= v->dims[i]; return n; }
static uint64_t numel_d(const uint64_t *d, int nd) { uint64_t n = 1; for (int i = 0; i < nd; i++) n *= d[i]; return n; }

static void var_release(Var *v) {
    if (v->kind == K_BUF && v->data && !v->borrowed) pool_free(v->data);
    v->data = NULL; v->borrowed = 0;
}

/* read one element of `id` at n-d index idx (sink coordinates of `id`) */
static float read_elem(const Oracle *o, uint32_t id, const uint64_t *idx_in) {
    uint64_t idx[MAXD], tmp[MAXD];
    const Var *v = &o->vars[id];
    memcpy(idx, idx_in, sizeof(uint64_t) * (size_t)(v->nd > 0 ? v->nd : 1));
    for (;;) {
        switch (v->kind) {
        case K_BUF: {
            uint64_t g = 0;
            for (int i = 0; i < v->nd; i++) g = g * v->dims[i] + idx[i];
            return v->data[g];
        }
        case K_CONST: return v->cval;
        case K_CONCAT:
            if (idx[v->cdim] > v->idx_end - 1 && v->idx_end > 0) { idx[v->cdim] -= v->idx_end; id = (uint32_t)v->cb; }
            else if (v->idx_end == 0) { id = (uint32_t)v->cb; }
            else id = (uint32_t)v->ca;
            v = &o->vars[id];
            break;
        case K_ALIAS:
            switch (v->acmd) {
            case A_VIEW: {
                uint64_t g = 0;
                for (int i = 0; i < v->nd; i++) g = g * v->dims[i] + idx[i];
                for (int i = v->src_nd - 1; i >= 0; i--) { tmp[i] = g % v->src_dims[i]; g /= v->src_dims[i]; }
                memcpy(idx, tmp, sizeof(uint64_t) * (size_t)v->src_nd);
                break;
            }
            case A_INDEX:
                for (int i = v->nd; i > v->adim; i--) idx[i] = idx[i - 1];
                idx[v->adim] = v->aindex;
                break;
            case A_PERMUTE:
                for (int i = 0; i < v->nd; i++) tmp[v->perm[i]] = idx[i];
                memcpy(idx, tmp, sizeof(uint64_t) * (size_t)v->nd);
                break;
            case A_BROADCAST: idx[v->adim] = 0; break;
            }
            id = (uint32_t)v->parent;
            v = &o->vars[id];
            break;
        default: return NAN;
        }
    }
}

/* contiguous copy of `id`; *owned tells the caller whether to free it */
static float *materialize(const Oracle *o, uint32_t id, int *owned) {
    const Var *v = &o->vars[id];
    uint64_t n = numel(v);
    if (v->kind == K_BUF) { *owned = 0; return v->data; }
    float *out = pool_alloc((size_t)n);
    *owned = 1;
    if (v->kind == K_CONST) {
        float c = v->cval;
#pragma omp parallel for schedule(static) if (n > 65536)
        for (uint64_t i = 0; i < n; i++) out[i] = c;
        return out;
    }
    /* common aliases get direct loops (same values as the generic path below, only faster) */
    if (v->kind == K_ALIAS && v->acmd == A_PERMUTE && v->nd == 2 && v->perm[0] == 1 && v->perm[1] == 0 &&
        o->vars[v->parent].kind == K_BUF) {
        const float *src = o->vars[v->parent].data;
        const uint64_t R = v->dims[0], C = v->dims[1]; /* out[r][c] = src[c][r], src is [C][R] */
#pragma omp parallel for schedule(static) collapse(2) if (n > 16384)
        for (uint64_t rb = 0; rb < R; rb += 32)
            for (uint64_t cb = 0; cb < C; cb += 32)
                for (uint64_t r = rb; r < rb + 32 && r < R; r++)
                    for (uint64_t c = cb; c < cb + 32 && c < C; c++) out[r * C + c] = src[c * R + r];
        return out;
    }
    if (v->kind == K_ALIAS && v->acmd == A_BROADCAST && v->nd == 2 && v->adim == 0) {
        const Var *p = &o->vars[v->parent];
        const float *row = NULL;
        if (p->kind == K_BUF) row = p->data;
        else if (p->kind == K_ALIAS && p->acmd == A_VIEW && o->vars[p->parent].kind == K_BUF) row = o->vars[p->parent].data;
        if (row) {
            const uint64_t R = v->dims[0], C = v->dims[1];
#pragma omp parallel for schedule(static) if (n > 16384)
            for (uint64_t r = 0; r < R; r++) memcpy(out + r * C, row, sizeof(float) * (size_t)C);
            return out;
        }
    }
    int nd = v->nd;
#pragma omp parallel for schedule(static) if (n > 16384)
    for (uint64_t i = 0; i < n; i++) {
        uint64_t idx[MAXD], g = i;
        for (int d = nd - 1; d >= 0; d--) { idx[d] = g % v->dims[d]; g /= v->dims[d]; }
        out[i] = read_elem(o, id, idx);
    }
    return out;
}

static int check_defined(Oracle *o, uint32_t id) {
    if (o->vars[id].kind == K_UNDEF) {
        snprintf(o->err, sizeof o->err, "oracle: id '%s' used before definition", o->names[id]);
        return -1;
    }
    return 0;
}

/* bind `id` to a buffer holding `data` (takes ownership) */
static void bind_buf(Oracle *o, uint32_t id, float *data, const uint64_t *dims, int nd) {
    Var *v = &o->vars[id];
    var_release(v);
    memset(v, 0, sizeof(*v));
    v->kind = K_BUF; v->nd = nd;
    memcpy(v->dims, dims, sizeof(uint64_t) * (size_t)nd);
    v->data = data;
}

/* ------------------------------------------------------------------ execution */
static int exec_proc(Oracle *o, Proc *p, int top);

static int exec_cmd(Oracle *o, Cmd *c) {
    Var *V = o->vars;
    o->cmds_executed++;
    switch (c->op) {
    case 1: { /* CreateMat: (re)upload every time it is executed (alloc.rs:5-12) */
        uint64_t n = numel_d(c->dims, c->nd);
        if (n != c->count) { snprintf(o->err, sizeof o->err, "oracle: CreateMat '%s' size mismatch", o->names[c->res]); return -1; }
        float *d = pool_alloc((size_t)n);
        memcpy(d, c->payload, sizeof(float) * (size_t)n);
        bind_buf(o, c->res, d, c->dims, c->nd);
        return 0;
    }
    case 2: {
        Var *v = &V[c->res];
        var_release(v); memset(v, 0, sizeof(*v));
        v->kind = K_CONST; v->cval = c->cval; v->nd = c->nd;
        memcpy(v->dims, c->dims, sizeof(uint64_t) * (size_t)c->nd);
        return 0;
    }
    case 3: case 4: case 5: case 6: {
        if (check_defined(o, c->a) || check_defined(o, c->b)) return -1;
        const Var *va = &V[c->a];
        uint64_t n = numel(va);
        uint64_t dims[MAXD]; int nd = va->nd;
        memcpy(dims, va->dims, sizeof dims);
        if (numel(&V[c->b]) != n && V[c->b].kind != K_CONST) {
            snprintf(o->err, sizeof o->err, "oracle: elementwise size mismatch %s vs %s", o->names[c->a], o->names[c->b]); return -1;
        }
        int oa = 0, ob = 0;
        /* a scalar constant is applied directly instead of being expanded to an array first */
        const int ca = V[c->a].kind == K_CONST, cb = V[c->b].kind == K_CONST;
        const float sa = V[c->a].cval, sb = V[c->b].cval;
        float *a = ca ? NULL : materialize(o, c->a, &oa);
        float *b = cb ? NULL : materialize(o, c->b, &ob);
        float *out = pool_alloc((size_t)n);
        const int mul = (c->op == 3 || c->op == 5);
        if (ca && cb) {
            const float r = mul ? sa * sb : sa + sb;
            for (uint64_t i = 0; i < n; i++) out[i] = r;
        } else if (ca || cb) {
            const float *x = ca ? b : a;
            const float k = ca ? sa : sb;
            if (mul) {
#pragma omp parallel for schedule(static) if (n > 65536)
                for (uint64_t i = 0; i < n; i++) out[i] = ca ? k * x[i] : x[i] * k;
            } else {
#pragma omp parallel for schedule(static) if (n > 65536)
                for (uint64_t i = 0; i < n; i++) out[i] = ca ? k + x[i] : x[i] + k;
            }
        } else if (mul) {
#pragma omp parallel for schedule(static) if (n > 65536)
            for (uint64_t i = 0; i < n; i++) out[i] = a[i] * b[i];
        } else {
#pragma omp parallel for schedule(static) if (n > 65536)
            for (uint64_t i = 0; i < n; i++) out[i] = a[i] + b[i];
        }
        if (oa) pool_free(a);
        if (ob) pool_free(b);
        bind_buf(o, c->res, out, dims, nd);
        return 0;
    }
    case 7: case 8: case 9: case 18: case 19: case 20: case 21: case 22: case 17: {
        if (check_defined(o, c->a)) return -1;
        const Var *va = &V[c->a];
        uint64_t n = numel(va);
        uint64_t dims[MAXD]; int nd = va->nd;
        memcpy(dims, va->dims, sizeof dims);
        int oa;
        float *a = materialize(o, c->a, &oa);
        float *out = pool_alloc((size_t)n);
        switch (c->op) {
#define LOOP(expr) _Pragma("omp parallel for schedule(static) if (n > 32768)") for (uint64_t i = 0; i < n; i++) { float x = a[i]; out[i] = (expr); }
        case 7: LOOP(x == 0.0f ? 1.0f : 0.0f) break;
        case 8: LOOP(x > 0.0f ? 1.0f : 0.0f) break;
        case 9: LOOP(x < 0.0f ? 1.0f : 0.0f) break;
        case 17: LOOP(x) break;
        case 18: LOOP(exp2f(x)) break;
        case 19: LOOP(log2f(x)) break;
        case 20: LOOP(sinf(x)) break;
        case 21: LOOP(1.0f / x) break;
        case 22: LOOP(sqrtf(fabsf(x))) break;
#undef LOOP
        }
        if (oa) pool_free(a);
        bind_buf(o, c->res, out, dims, nd);
        return 0;
    }
    case 10: { /* Sum over the last axis of a 2-d tensor */
        if (check_defined(o, c->a)) return -1;
        const Var *va = &V[c->a];
        if (va->nd != 2) { snprintf(o->err, sizeof o->err, "oracle: Sum needs a 2-d input ('%s')", o->names[c->a]); return -1; }
        uint64_t vs = va->dims[0], rs = va->dims[1];
        int oa;
        float *a = materialize(o, c->a, &oa);
        float *out = pool_alloc((size_t)vs);
        int f64 = o->f64_acc;
#pragma omp parallel for schedule(static) if (vs * rs > 65536)
        for (uint64_t x = 0; x < vs; x++) {
            const float *row = a + x * rs;
            if (f64) { double s = 0; for (uint64_t y = 0; y < rs; y++) s += row[y]; out[x] = (float)s; }
            else { float s = 0; for (uint64_t y = 0; y < rs; y++) s += row[y]; out[x] = s; }
        }
        if (oa) pool_free(a);
        uint64_t dims[1] = { vs };
        bind_buf(o, c->res, out, dims, 1);
        return 0;
    }
    case 28: { /* Max over the last axis of a 2-d tensor (IR extension; fmaxf semantics: a NaN operand is ignored) */
        if (check_defined(o, c->a)) return -1;
        const Var *va = &V[c->a];
        if (va->nd != 2) { snprintf(o->err, sizeof o->err, "oracle: Max needs a 2-d input ('%s')", o->names[c->a]); return -1; }
        uint64_t vs = va->dims[0], rs = va->dims[1];
        int oa;
        float *a = materialize(o, c->a, &oa);
        float *out = pool_alloc((size_t)vs);
#pragma omp parallel for schedule(static) if (vs * rs > 65536)
        for (uint64_t x = 0; x < vs; x++) {
            const float *row = a + x * rs;
            float m = -INFINITY;
            for (uint64_t y = 0; y < rs; y++) m = fmaxf(m, row[y]);
            out[x] = m;
        }
        if (oa) pool_free(a);
        uint64_t dims[1] = { vs };
        bind_buf(o, c->res, out, dims, 1);
        return 0;
    }
    case 11: { /* DotProduct: [M,K] x [K,N], k ascending */
        if (check_defined(o, c->a) || check_defined(o, c->b)) return -1;
        const Var *va = &V[c->a], *vb = &V[c->b];
        if (va->nd != 2 || vb->nd != 2 || va->dims[1] != vb->dims[0]) {
            snprintf(o->err, sizeof o->err, "oracle: DotProduct shape mismatch"); return -1;
        }
        uint64_t M = va->dims[0], K = va->dims[1], N = vb->dims[1];
        int oa, ob;
        float *a = materialize(o, c->a, &oa);
        float *b = materialize(o, c->b, &ob);
        float *out = pool_alloc((size_t)(M * N));
#pragma omp parallel for schedule(static) if (M * N > 65536)
        for (uint64_t i = 0; i < M * N; i++) out[i] = 0.0f;
        int f64 = o->f64_acc;
        if (f64) {
#pragma omp parallel for schedule(static)
            for (uint64_t i = 0; i < M; i++) {
                double *acc = calloc((size_t)N, sizeof(double));
                for (uint64_t k = 0; k < K; k++) { double av = a[i * K + k]; const float *br = b + k * N; for (uint64_t j = 0; j < N; j++) acc[j] += av * br[j]; }
                for (uint64_t j = 0; j < N; j++) out[i * N + j] = (float)acc[j];
                free(acc);
            }
        } else {
            /* tiles of 8 rows x 512 columns; inside a tile k runs outermost, so every out[i][j] still
             * accumulates its products in ascending k (the reference's order), while a row of B is
             * reused by the 8 rows of the tile instead of being streamed from memory for each of them */
            const uint64_t TI = 8, TJ = 512;
            const uint64_t nti = (M + TI - 1) / TI, ntj = (N + TJ - 1) / TJ;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
            for (uint64_t ti = 0; ti < nti; ti++)
                for (uint64_t tj = 0; tj < ntj; tj++) {
                    const uint64_t i0 = ti * TI, i1 = i0 + TI < M ? i0 + TI : M;
                    const uint64_t j0 = tj * TJ, j1 = j0 + TJ < N ? j0 + TJ : N;
                    for (uint64_t k = 0; k < K; k++) {
                        const float *br = b + k * N;
                        for (uint64_t i = i0; i < i1; i++) {
                            const float av = a[i * K + k];
                            float *cr = out + i * N;
                            for (uint64_t j = j0; j < j1; j++) cr[j] += av * br[j];
                        }
                    }
                }
        }
        if (oa) pool_free(a);
        if (ob) pool_free(b);
        uint64_t dims[2] = { M, N };
        bind_buf(o, c->res, out, dims, 2);
        return 0;
    }
    case 29: { /* BatchDot (extension): [B,M,K] x [B,K,N] -> [B,M,N], every slice as DotProduct: k ascending, fp32 */
        if (check_defined(o, c->a) || check_defined(o, c->b)) return -1;
        const Var *va = &V[c->a], *vb = &V[c->b];
        if (va->nd != 3 || vb->nd != 3 || va->dims[0] != vb->dims[0] || va->dims[2] != vb->dims[1]) {
            snprintf(o->err, sizeof o->err, "oracle: BatchDot shape mismatch"); return -1;
        }
        uint64_t B = va->dims[0], M = va->dims[1], K = va->dims[2], N = vb->dims[2];
        int oa, ob;
        float *a = materialize(o, c->a, &oa);
        float *b = materialize(o, c->b, &ob);
        float *out = pool_alloc((size_t)(B * M * N));
#pragma omp parallel for schedule(static) collapse(2) if (B * M * N * K > 65536)
        for (uint64_t s = 0; s < B; s++)
            for (uint64_t i = 0; i < M; i++) {
                float *cr = out + (s * M + i) * N;
                for (uint64_t j = 0; j < N; j++) cr[j] = 0.0f;
                for (uint64_t k = 0; k < K; k++) {
                    const float av = a[(s * M + i) * K + k];
                    const float *br = b + (s * K + k) * N;
                    if (o->f64_acc) { for (uint64_t j = 0; j < N; j++) cr[j] = (float)((double)cr[j] + (double)av * (double)br[j]); }
                    else for (uint64_t j = 0; j < N; j++) cr[j] += av * br[j];
                }
            }
        if (oa) pool_free(a);
        if (ob) pool_free(b);
        uint64_t dims[3] = { B, M, N };
        bind_buf(o, c->res, out, dims, 3);
        return 0;
    }
    case 12: case 13: case 15: case 16: { /* aliases */
        if (check_defined(o, c->a)) return -1;
        Var nv; memset(&nv, 0, sizeof nv);
        const Var *va = &V[c->a];
        nv.kind = K_ALIAS; nv.parent = (int)c->a;
        if (c->a == c->res) { snprintf(o->err, sizeof o->err, "oracle: alias onto itself ('%s')", o->names[c->a]); return -1; }
        if (c->op == 12) {
            nv.acmd = A_VIEW; nv.nd = c->nd; memcpy(nv.dims, c->dims, sizeof nv.dims);
            nv.src_nd = va->nd; memcpy(nv.src_dims, va->dims, sizeof nv.src_dims);
            if (numel_d(nv.dims, nv.nd) != numel(va)) { snprintf(o->err, sizeof o->err, "oracle: View size mismatch"); return -1; }
        } else if (c->op == 13) {
            if ((int)c->dim >= va->nd || c->index >= va->dims[c->dim]) { snprintf(o->err, sizeof o->err, "oracle: Index out of range"); return -1; }
            nv.acmd = A_INDEX; nv.adim = (int)c->dim; nv.aindex = c->index; nv.nd = va->nd - 1;
            for (int i = 0, j = 0; i < va->nd; i++) if (i != (int)c->dim) nv.dims[j++] = va->dims[i];
        } else if (c->op == 15) {
            if (c->nd != va->nd) { snprintf(o->err, sizeof o->err, "oracle: Permute rank mismatch"); return -1; }
            nv.acmd = A_PERMUTE; nv.nd = va->nd;
            for (int i = 0; i < va->nd; i++) { nv.perm[i] = (int)c->perm[i]; nv.dims[i] = va->dims[c->perm[i]]; }
        } else {
            if ((int)c->dim >= va->nd) { snprintf(o->err, sizeof o->err, "oracle: Broadcast dim out of range"); return -1; }
            nv.acmd = A_BROADCAST; nv.adim = (int)c->dim; nv.nd = va->nd;
            memcpy(nv.dims, va->dims, sizeof nv.dims); nv.dims[c->dim] = c->count;
        }
        var_release(&V[c->res]);
        V[c->res] = nv;
        return 0;
    }
    case 14: {
        if (check_defined(o, c->a) || check_defined(o, c->b)) return -1;
        if (c->res == c->a || c->res == c->b) { snprintf(o->err, sizeof o->err, "oracle: Res id can't be the same as a and b id at Concat"); return -1; }
        const Var *va = &V[c->a], *vb = &V[c->b];
        if (va->nd != vb->nd || (int)c->dim >= va->nd) { snprintf(o->err, sizeof o->err, "oracle: Concat rank mismatch"); return -1; }
        Var nv; memset(&nv, 0, sizeof nv);
        nv.kind = K_CONCAT; nv.ca = (int)c->a; nv.cb = (int)c->b; nv.cdim = (int)c->dim;
        nv.idx_end = va->dims[c->dim]; nv.nd = va->nd;
        memcpy(nv.dims, va->dims, sizeof nv.dims);
        nv.dims[c->dim] += vb->dims[c->dim];
        var_release(&V[c->res]);
        V[c->res] = nv;
        return 0;
    }
    case 23: {
        for (;;) {
            if (check_defined(o, c->a)) return -1;
            uint64_t z[MAXD] = { 0 };
            float cv = read_elem(o, c->a, z);
            if (!(cv != 0.0f)) break;
            if (exec_proc(o, &c->block, 0)) return -1;
            if (o->stop) return 0;
        }
        return 0;
    }
    case 24: {
        uint64_t z[MAXD] = { 0 };
        for (uint32_t k = 0; k < c->ncond; k++) {
            if (check_defined(o, c->cond_ids[k])) return -1;
            if (read_elem(o, c->cond_ids[k], z) == 1.0f) return exec_proc(o, &c->cond_blocks[k], 0);
        }
        if (c->has_else) return exec_proc(o, &c->else_block, 0);
        return 0;
    }
    case 25: o->stop = 1; return 0;
    case 26: return 0;
    case 27: {
        if (check_defined(o, c->a)) return -1;
        if (V[c->a].kind != K_BUF) { snprintf(o->err, sizeof o->err, "oracle: AllReduce target must be a buffer"); return -1; }
        if (o->allreduce) o->allreduce(V[c->a].data, numel(&V[c->a]), o->allreduce_user);
        return 0;
    }
    }
    snprintf(o->err, sizeof o->err, "oracle: unhandled opcode %u", c->op);
    return -1;
}

static int exec_proc(Oracle *o, Proc *p, int top) {
    for (uint32_t i = 0; i < p->n; i++) {
        if (exec_cmd(o, &p->cmds[i])) return -1;
        if (o->stop) return 0;
        if (top) {
            /* release buffers whose last textual use is behind us */
            Cmd *c = &p->cmds[i];
            uint32_t ids[3] = { c->a, c->b, c->res };
            for (int k = 0; k < 3; k++) {
                uint32_t id = ids[k];
                Var *v = &o->vars[id];
                if (v->kind == K_BUF && !o->is_dep[id] && o->last_use[id] <= i && v->data) {
                    var_release(v); v->kind = K_UNDEF;
                }
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ public API */
static void clear_results(Oracle *o) {
    for (uint32_t i = 0; i < o->n_res; i++) { free(o->res_names[i]); free(o->res_data[i]); }
    free(o->res_names); free(o->res_data); free(o->res_dims); free(o->res_nd);
    o->res_names = NULL; o->res_data = NULL; o->res_dims = NULL; o->res_nd = NULL; o->n_res = 0;
}

static void clear_program(Oracle *o) {
    for (uint32_t i = 0; i < o->n_ids; i++) { var_release(&o->vars[i]); free(o->names[i]); }
    free(o->vars); free(o->names); free(o->dep); free(o->is_dep); free(o->last_use);
    free_proc(&o->main);
    o->vars = NULL; o->names = NULL; o->dep = NULL; o->is_dep = NULL; o->last_use = NULL; o->n_ids = 0; o->n_dep = 0;
}

void *oracle_create(void) {
    Oracle *o = calloc(1, sizeof(Oracle));
    const char *e = getenv("ADB_ORACLE_F64ACC");
    o->f64_acc = (e && e[0] == '1');
    return o;
}

void oracle_set_f64_acc(void *h, int on) { ((Oracle *)h)->f64_acc = on; }
void oracle_set_allreduce(void *h, allreduce_fn fn, void *user) { Oracle *o = h; o->allreduce = fn; o->allreduce_user = user; }
uint64_t oracle_cmds_executed(void *h) { return ((Oracle *)h)->cmds_executed; }
/* Threads of the OpenMP loops.  A launcher may export OMP_NUM_THREADS=1 to its children (torch.distributed.run
 * does); a caller that times the oracle as the CPU baseline sets the count it means and reports what it got. */
#ifdef _OPENMP
#include <omp.h>
int oracle_set_threads(int n) { if (n > 0) omp_set_num_threads(n); return omp_get_max_threads(); }
#else
int oracle_set_threads(int n) { (void)n; return 1; }
#endif

void oracle_destroy(void *h) {
    Oracle *o = h;
    if (!o) return;
    clear_program(o); clear_results(o);
    free(o);
}

const char *oracle_last_error(void *h) { return ((Oracle *)h)->err; }

int oracle_execute(void *h, const uint8_t *blob, size_t nbytes) {
    Oracle *o = h;
    clear_program(o); clear_results(o);
    o->err[0] = 0; o->stop = 0; o->cmds_executed = 0;
    Rd r = { blob, blob, blob + nbytes, 0 };
    uint32_t magic = r32(&r), version = r32(&r);
    (void)r32(&r);
    if (magic != 0x52494441u || version != 1) { snprintf(o->err, sizeof o->err, "oracle: bad magic/version"); return -1; }
    o->n_ids = r32(&r);
    if (r.bad || o->n_ids > (1u << 28)) { snprintf(o->err, sizeof o->err, "oracle: bad id table"); o->n_ids = 0; return -1; }
    o->names = calloc(o->n_ids ? o->n_ids : 1, sizeof(char *));
    o->vars = calloc(o->n_ids ? o->n_ids : 1, sizeof(Var));
    o->is_dep = calloc(o->n_ids ? o->n_ids : 1, 1);
    o->last_use = calloc(o->n_ids ? o->n_ids : 1, sizeof(uint32_t));
    for (uint32_t i = 0; i < o->n_ids; i++) {
        uint16_t n = r16(&r);
        if (r.p + n > r.end) { snprintf(o->err, sizeof o->err, "oracle: truncated id table"); return -1; }
        o->names[i] = malloc((size_t)n + 1);
        memcpy(o->names[i], r.p, n); o->names[i][n] = 0; r.p += n;
    }
    o->n_dep = r32(&r);
    if (r.bad || o->n_dep > o->n_ids) { snprintf(o->err, sizeof o->err, "oracle: bad dep list"); o->n_dep = 0; return -1; }
    o->dep = calloc(o->n_dep ? o->n_dep : 1, sizeof(uint32_t));
    for (uint32_t i = 0; i < o->n_dep; i++) {
        o->dep[i] = r32(&r);
        if (o->dep[i] >= o->n_ids) { snprintf(o->err, sizeof o->err, "oracle: dep id out of range"); return -1; }
        o->is_dep[o->dep[i]] = 1;
    }
    if (parse_proc(o, &r, &o->main, 0)) return -1;
    scan_uses(o, &o->main, 1, 0);
    for (uint32_t i = 0; i < o->n_dep; i++) o->last_use[o->dep[i]] = UINT32_MAX; /* read back at the end */
    propagate_alias(o, &o->main);
    if (exec_proc(o, &o->main, 1)) return -1;

    /* read-back of dep-list ids (device.rs:82-87) */
    o->res_names = calloc(o->n_dep ? o->n_dep : 1, sizeof(char *));
    o->res_data = calloc(o->n_dep ? o->n_dep : 1, sizeof(float *));
    o->res_dims = calloc(o->n_dep ? o->n_dep : 1, sizeof(uint64_t[MAXD]));
    o->res_nd = calloc(o->n_dep ? o->n_dep : 1, sizeof(int));
    for (uint32_t i = 0; i < o->n_dep; i++) {
        uint32_t id = o->dep[i];
        Var *v = &o->vars[id];
        if (v->kind == K_UNDEF) continue;
        int owned;
        float *d = materialize(o, id, &owned);
        uint64_t n = numel(v);
        float *copy = malloc(sizeof(float) * (size_t)(n ? n : 1));
        memcpy(copy, d, sizeof(float) * (size_t)n);
        if (owned) pool_free(d);
        uint32_t k = o->n_res++;
        o->res_names[k] = strdup(o->names[id]);
        o->res_data[k] = copy;
        o->res_nd[k] = v->nd;
        memcpy(o->res_dims[k], v->dims, sizeof(uint64_t) * MAXD);
    }
    /* working set is no longer needed */
    for (uint32_t i = 0; i < o->n_ids; i++) { var_release(&o->vars[i]); o->vars[i].kind = K_UNDEF; }
    return 0;
}

/* 0 = found, 1 = none (the id was not kept), mirrors ValueData::none() */
int oracle_get_tensor(void *h, const char *id, const float **data, const uint64_t **dims, uint32_t *ndim) {
    Oracle *o = h;
    for (uint32_t i = 0; i < o->n_res; i++)
        if (strcmp(o->res_names[i], id) == 0) {
            *data = o->res_data[i]; *dims = o->res_dims[i]; *ndim = (uint32_t)o->res_nd[i];
            return 0;
        }
    return 1;
}
