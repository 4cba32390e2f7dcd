/* Test infrastructure only: exposes the double-precision router oracle that the reference keeps as a static function inside
 * its own test (tests/gpu_router_test.c:62-79) by compiling that test file where it lies, with its main renamed. Built by
 * `make ref` into _ref/libref_router.so; nothing of the reference is copied. */
#define main omega_router_test_main_unused
#include "gpu_router_test.c"
#undef main

void ref_router_oracle(const float *x, const float *nw, const uint16_t *gate_bf16, int norm_topk, double *xn, double *logits,
                       uint32_t *ids, double *w, double *margin) {
    static Case c;
    memcpy(c.x, x, sizeof c.x); memcpy(c.nw, nw, sizeof c.nw);
    c.gate = (uint16_t *)gate_bf16;
    oracle_fill(&c, norm_topk);
    memcpy(xn, c.xn, sizeof c.xn); memcpy(logits, c.logits, sizeof c.logits);
    memcpy(ids, c.ids, sizeof c.ids); memcpy(w, c.w, sizeof c.w); *margin = c.margin;
}
unsigned ref_router_hidden(void) { return H; }
unsigned ref_router_experts(void) { return NE; }
unsigned ref_router_topk(void) { return TK; }
float ref_router_eps(void) { return EPS; }
