// Downstream use of the installed package: the reference's include path and template names.
#include <cstdio>

#include "flash_attn/flash_api.cuh"

int main() {
  int compiled = 0;
  for (int d : {32, 64, 96, 128, 192, 256}) compiled += tfa::isHeadDimCompiled(d) ? 1 : 0;
  std::printf("head dims compiled: %d\n", compiled);
  // never called at run time here (no device needed to link): takes the address so the template is instantiated
  auto fn = &tfa::flashAttn<__nv_bfloat16>;
  return fn == nullptr;
}
