/*
 * b200moe_plan.h: the top-k routing plan (token-to-expert grouping) and its wire serialisers.
 *
 * Drop-in for the reference's plan units (declared in src/cudapp_native.h:33-38; contracts in
 * om/moe/README.md and om/moe/moe_plan.om). Calling convention ("ABI1"): uint32_t status = fn(&result, views...);
 * every view is (pointer, element count) with the exact declared length; status 0 = ran (the unit's own return
 * code is in *result), 32 = a view has the wrong length, is NULL, misaligned or overlaps another, 33 = re-entered.
 * *result is written only when status is 0. A unit that refuses (result != 0) leaves every output byte unchanged.
 *
 * omega_moe_plan computes the plan ON THE GPU (histogram, exclusive scan, stable scatter; see
 * omega_gpu_moe_plan_async for the device-resident form the MoE layer uses) and copies the logical words back;
 * it fails with status 14 when no CUDA device is usable. The four serialisers only re-encode small host arrays
 * into the device wire formats (u32 maps, 32-byte segment records, launch words) and are plain host code, as in
 * the reference.
 */
#ifndef B200MOE_PLAN_H
#define B200MOE_PLAN_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
#define OMEGA_OK 0u
#define OMEGA_BAD_ARG 32u
#define OMEGA_REENTRY 33u

/* src/cudapp_native.h:33. cfg u64[8] = {1, tokens <= 128, slots <= 8, experts 1..256, shared id == experts, work
 * capacity <= 1152, segment capacity <= 257, map capacity <= 1160}; ids u64[1024] token-major, 0xFFFFFFFF = absent;
 * work u64[10368] (9 words per row: expert, source row, token, slot, weight slot, segment offset, segment count,
 * destination token*(slots+1)+slot, order); seg u64[1028] ({expert, offset, count, shared} per non-empty expert,
 * the shared expert last); maps u64[2320] (X at 0, Y at 1160, 8 zero entries after the last row of each);
 * meta u64[8] = {work rows, segments, routed rows, tokens, 1, 0, 0, 0}. result: 0, 1 cfg, 2 id, 3 capacity. */
uint32_t omega_moe_plan(uint64_t *result, const void *cfg, uint64_t cfg_n, const void *ids, uint64_t ids_n, void *work, uint64_t work_n,
                        void *seg, uint64_t seg_n, void *maps, uint64_t maps_n, void *meta, uint64_t meta_n);
/* src/cudapp_native.h:34: 16 request words -> 64 bytes of GROUP launch words (om/moe/moe_group.om:55-101). */
uint32_t omega_moe_group(uint64_t *result, const void *req, uint64_t req_n, void *words, uint64_t words_n);
/* src/cudapp_native.h:35: 4096 bytes of LE u32 picks, n active -> ids u64[1024] (om/moe/moe_ids32.om). */
uint32_t omega_moe_ids32(uint64_t *result, const void *src, uint64_t src_n, uint64_t n, void *ids, uint64_t ids_n);
/* src/cudapp_native.h:36: meta u64[8], maps u64[2320] -> 9280 bytes of LE u32 maps (om/moe/moe_maps32.om). */
uint32_t omega_moe_maps32(uint64_t *result, const void *meta, uint64_t meta_n, const void *maps, uint64_t maps_n, void *out, uint64_t out_n);
/* src/cudapp_native.h:37: seg u64[1028], meta u64[8], directory u64[514] -> 8224 bytes of 32-byte segment records. */
uint32_t omega_moe_segs32(uint64_t *result, const void *seg, uint64_t seg_n, const void *meta, uint64_t meta_n, const void *dir, uint64_t dir_n,
                          void *out, uint64_t out_n);
/* src/cudapp_native.h:38: cfg u64[8] -> windows u64[1024] (8 per window), meta u64[4] (om/moe/moe_windows.om). */
uint32_t omega_moe_windows(uint64_t *result, const void *cfg, uint64_t cfg_n, void *windows, uint64_t windows_n, void *meta, uint64_t meta_n);
#ifdef __cplusplus
}
#endif
#endif
