/*
 * The reference engine's library boundary, kept verbatim: the three functions engine/libllada.cu:13-52 exports and
 * server/server.py:62-71 binds over ctypes. A drop-in libllada.so is the reference's own libllada.cu built with
 * attn_shim.cuh in place of attn.cu (oracle/Makefile's `dropin` target does exactly that); this repository does not
 * re-implement the model forward pass behind these calls.
 */
#ifndef LIBLLADA_H
#define LIBLLADA_H
#ifdef __cplusplus
extern "C" {
#endif

/* engine/libllada.cu:15 — loads the packed model in `dir`, returns an opaque handle that is never freed. */
void* llada_init(const char* dir, int max_ctx);

/* engine/libllada.cu:26 — generates after `prompt`; `out` receives up to out_cap ids; on_block (may be NULL) is called
 * on the caller's thread with every decoded block; steps is clamped to [1, 32]; returns the number of ids written. */
int llada_generate(void* h, const int* prompt, int n, int max_new, float threshold, float editing_threshold,
                   int max_post_steps, int steps, int* out, int out_cap, void (*on_block)(const int*, int, void*),
                   void* user);

/* engine/libllada.cu:45 — s[0..6] = steps, blocks, commits, reused blocks, weight GB, kv GB, max context. */
void llada_stats(void* h, double* s);

#ifdef __cplusplus
}
#endif
#endif
