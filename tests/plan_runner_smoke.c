/* Compiles against the plan runner's C header and exercises its error paths (no GPU needed): a missing plan file, a
 * file that is not a plan, and index checks on a null-free API surface. Prints one line per check. */
#include <stdio.h>
#include <string.h>

#include "fd_plan_runner.h"

int main(int argc, char** argv) {
  if (argc < 4) return 2;
  const char* kernels = argv[1];
  void* p = fdplan_load(argv[2], kernels);                 /* does not exist */
  printf("missing: %s | %s\n", p == NULL ? "null" : "loaded", fdplan_last_error());
  p = fdplan_load(argv[3], kernels);                       /* exists, wrong magic */
  printf("garbage: %s | %s\n", p == NULL ? "null" : "loaded", fdplan_last_error());
  p = fdplan_load(argv[3], "/nonexistent/libfdb200_kernels.so");
  printf("nolib: %s | %s\n", p == NULL ? "null" : "loaded", strlen(fdplan_last_error()) > 0 ? "message" : "empty");
  return 0;
}
