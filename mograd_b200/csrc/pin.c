/* Keeps the library mapped for the life of the process: a host runtime whose
 * destructors run after it dlclose()d the kernel library must not jump into
 * unmapped text.  Same purpose as mograd/runtime/gpu/kernels/pin.c:1-21. */
#define _GNU_SOURCE
#include <dlfcn.h>

static void mgb_pin_anchor(void) {}

__attribute__((constructor)) static void mgb_pin_self(void) {
  Dl_info info;
  if (dladdr((void*)&mgb_pin_anchor, &info) && info.dli_fname)
    (void)dlopen(info.dli_fname, RTLD_NOW | RTLD_NODELETE);
}
