// Process-wide switch of programmatic dependent launches (see tf_pdl_sync / tf_launch in common.cuh).
#include "common.cuh"

int g_tf_pdl = 0;

// on != 0: every kernel of this library is launched with the programmatic-stream-serialization
// attribute, in eager launches and under stream capture alike.  Returns the previous setting.
TF_API int tf_set_pdl(int on) {
  const int old = g_tf_pdl;
  g_tf_pdl = on ? 1 : 0;
  return old;
}

TF_API int tf_get_pdl() { return g_tf_pdl; }
