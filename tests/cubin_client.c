/* A client of the library that loads and launches the kernel ITSELF, the way rocMLIR's clients treat its code object
 * (MIGraphX: mlirGetBinary + mlirGetKernelAttrs, then hipModuleLoadData / hipModuleLaunchKernel): it asks the
 * library for the sm_100a cubin and for the launch description of one fp16 GEMM, loads the image with
 * cuModuleLoadData, launches the named kernel with cuLaunchKernelEx, and compares the result bit for bit with what
 * rbGemm writes for the same buffers. Plain C, no CUDA headers: the driver and the library are opened with dlopen.
 *
 *   cc -O1 -o cubin_client cubin_client.c -ldl && ./cubin_client <path to librocmlir_b200.so>  ->  "MATCH ..." */
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "rocmlir_b200.h"

typedef int CUresult;
typedef int CUdevice;
typedef void *CUcontext, *CUmodule, *CUfunction, *CUstream;
typedef unsigned long long CUdeviceptr;
/* cuda.h: CUlaunchAttribute is {id, pad[4], 64-byte value union}; CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION = 4 */
typedef struct { int id; char pad[4]; union { struct { unsigned x, y, z; } clusterDim; char bytes[64]; } value; } LaunchAttr;
typedef struct { unsigned gx, gy, gz, bx, by, bz, smem; CUstream stream; LaunchAttr *attrs; unsigned nattrs; } LaunchConfig;
#define CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES 8

#define CHECK(x) do { int r_ = (x); if (r_ != 0) { fprintf(stderr, "%s failed: %d\n", #x, r_); return 1; } } while (0)
/* declares a function pointer `var` for symbol `name` of `lib` */
#define SYM(lib, ret, var, name, args) ret (*var) args = (ret (*) args)dlsym(lib, #name); \
  if (!var) { fprintf(stderr, "missing %s\n", #name); return 1; }

static uint16_t f16_of_small_int(int v) {   /* exact for |v| <= 2048 */
  if (v == 0) return 0;
  uint16_t sign = v < 0 ? 0x8000 : 0;
  unsigned a = v < 0 ? -v : v;
  int e = 0;
  while ((a >> (e + 1)) != 0) ++e;
  unsigned mant = (a << (10 - e)) & 0x3ff;
  return sign | (uint16_t)((e + 15) << 10) | (uint16_t)mant;
}

int main(int argc, char **argv) {
  if (argc < 2) { fprintf(stderr, "usage: %s <librocmlir_b200.so>\n", argv[0]); return 2; }
  void *cu = dlopen("libcuda.so.1", RTLD_NOW), *rb = dlopen(argv[1], RTLD_NOW);
  if (!cu || !rb) { fprintf(stderr, "dlopen: %s\n", dlerror()); return 1; }
  SYM(cu, CUresult, cuInit, cuInit, (unsigned))
  SYM(cu, CUresult, cuDeviceGet, cuDeviceGet, (CUdevice *, int))
  SYM(cu, CUresult, cuDevicePrimaryCtxRetain, cuDevicePrimaryCtxRetain, (CUcontext *, CUdevice))
  SYM(cu, CUresult, cuCtxSetCurrent, cuCtxSetCurrent, (CUcontext))
  SYM(cu, CUresult, cuMemAlloc_v2, cuMemAlloc_v2, (CUdeviceptr *, size_t))
  SYM(cu, CUresult, cuMemcpyHtoD_v2, cuMemcpyHtoD_v2, (CUdeviceptr, const void *, size_t))
  SYM(cu, CUresult, cuMemcpyDtoH_v2, cuMemcpyDtoH_v2, (void *, CUdeviceptr, size_t))
  SYM(cu, CUresult, cuMemsetD8_v2, cuMemsetD8_v2, (CUdeviceptr, unsigned char, size_t))
  SYM(cu, CUresult, cuModuleLoadData, cuModuleLoadData, (CUmodule *, const void *))
  SYM(cu, CUresult, cuModuleGetFunction, cuModuleGetFunction, (CUfunction *, CUmodule, const char *))
  SYM(cu, CUresult, cuFuncSetAttribute, cuFuncSetAttribute, (CUfunction, int, int))
  SYM(cu, CUresult, cuLaunchKernelEx, cuLaunchKernelEx, (const LaunchConfig *, CUfunction, void **, void **))
  SYM(cu, CUresult, cuCtxSynchronize, cuCtxSynchronize, (void))
  SYM(rb, RbStatus, p_rbGetKernelBinary, rbGetKernelBinary, (const void **, size_t *))
  SYM(rb, RbStatus, p_rbGemmEncodeLaunch, rbGemmEncodeLaunch, (const RbGemmProblem *, const RbEpilogue *, const void *, const void *, void *, RbKernelLaunch *))
  SYM(rb, RbStatus, p_rbGemm, rbGemm, (const RbGemmProblem *, const RbEpilogue *, const void *, const void *, void *, void *, size_t, void *))
  SYM(rb, RbStatus, p_rbReadKernelStatus, rbReadKernelStatus, (uint32_t *, int))
  SYM(rb, const char *, p_rbGetLastError, rbGetLastError, (void))

  CUdevice dev; CUcontext ctx;
  CHECK(cuInit(0)); CHECK(cuDeviceGet(&dev, 0)); CHECK(cuDevicePrimaryCtxRetain(&ctx, dev)); CHECK(cuCtxSetCurrent(ctx));

  /* one batch, M = 384 (a CTA pair and a half), N = 520 (ragged last tile), K = 512; integer-valued data: exact */
  RbGemmProblem p; memset(&p, 0, sizeof(p));
  p.g = 1; p.m = 384; p.n = 520; p.k = 512;   /* eight K blocks: short enough that the library does not cut K into ranges */ p.ab_type = RB_F16; p.c_type = RB_F16;
  size_t na = (size_t)p.m * p.k, nb = (size_t)p.k * p.n, nc = (size_t)p.m * p.n;
  uint16_t *ha = malloc(na * 2), *hb = malloc(nb * 2), *c1 = malloc(nc * 2), *c2 = malloc(nc * 2);
  unsigned s = 12345;
  for (size_t i = 0; i < na; ++i) { s = s * 1664525u + 1013904223u; ha[i] = f16_of_small_int((int)((s >> 16) % 10) - 5); }
  for (size_t i = 0; i < nb; ++i) { s = s * 1664525u + 1013904223u; hb[i] = f16_of_small_int((int)((s >> 16) % 10) - 5); }
  CUdeviceptr da, db, dc1, dc2;
  CHECK(cuMemAlloc_v2(&da, na * 2)); CHECK(cuMemAlloc_v2(&db, nb * 2)); CHECK(cuMemAlloc_v2(&dc1, nc * 2)); CHECK(cuMemAlloc_v2(&dc2, nc * 2));
  CHECK(cuMemcpyHtoD_v2(da, ha, na * 2)); CHECK(cuMemcpyHtoD_v2(db, hb, nb * 2));
  CHECK(cuMemsetD8_v2(dc1, 0xEE, nc * 2)); CHECK(cuMemsetD8_v2(dc2, 0x11, nc * 2));

  /* the library's own launch */
  if (p_rbGemm(&p, NULL, (void *)da, (void *)db, (void *)dc1, NULL, 0, NULL) != RB_SUCCESS) { fprintf(stderr, "rbGemm: %s\n", p_rbGetLastError()); return 1; }

  /* the client's launch of the same kernel out of the cubin */
  const void *image; size_t image_size; RbKernelLaunch kl;
  if (p_rbGetKernelBinary(&image, &image_size) != RB_SUCCESS) return 1;
  if (p_rbGemmEncodeLaunch(&p, NULL, (void *)da, (void *)db, (void *)dc2, &kl) != RB_SUCCESS) { fprintf(stderr, "encode: %s\n", p_rbGetLastError()); return 1; }
  CUmodule mod; CUfunction fn;
  CHECK(cuModuleLoadData(&mod, image));
  CHECK(cuModuleGetFunction(&fn, mod, kl.symbol));
  CHECK(cuFuncSetAttribute(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)kl.dynamic_smem));
  LaunchAttr attr; memset(&attr, 0, sizeof(attr));
  attr.id = 4; attr.value.clusterDim.x = kl.cluster; attr.value.clusterDim.y = 1; attr.value.clusterDim.z = 1;
  LaunchConfig lc; memset(&lc, 0, sizeof(lc));
  lc.gx = kl.grid; lc.gy = lc.gz = 1; lc.bx = kl.block; lc.by = lc.bz = 1; lc.smem = kl.dynamic_smem;
  lc.attrs = &attr; lc.nattrs = 1;
  void *params[4];
  for (unsigned i = 0; i < kl.param_count; ++i) params[i] = kl.params + kl.param_offset[i];
  CHECK(cuLaunchKernelEx(&lc, fn, params, NULL));
  CHECK(cuCtxSynchronize());
  uint32_t status = 0;
  if (p_rbReadKernelStatus(&status, 1) != RB_SUCCESS || status != 0) { fprintf(stderr, "kernel status %u\n", status); return 1; }
  CHECK(cuMemcpyDtoH_v2(c1, dc1, nc * 2)); CHECK(cuMemcpyDtoH_v2(c2, dc2, nc * 2));
  if (memcmp(c1, c2, nc * 2) != 0) { printf("DIFFER\n"); return 1; }
  /* and one element against the definition */
  long acc = 0;
  for (int k = 0; k < p.k; ++k) {
    uint16_t x = ha[(size_t)7 * p.k + k], y = hb[(size_t)k * p.n + 519];
    int xi = (x & 0x3ff) | 0x400, yi = (y & 0x3ff) | 0x400;   /* decode the small integers again */
    int xe = ((x >> 10) & 31) - 25, ye = ((y >> 10) & 31) - 25;
    long xv = x & 0x7fff ? (xe >= 0 ? (long)xi << xe : (long)xi >> -xe) : 0, yv = y & 0x7fff ? (ye >= 0 ? (long)yi << ye : (long)yi >> -ye) : 0;
    acc += (x & 0x8000 ? -xv : xv) * (y & 0x8000 ? -yv : yv);
  }
  printf("MATCH image %zu bytes, kernel %s, grid %u x block %u, cluster %u, smem %u, C[7][519] = %ld (f16 bits %04x)\n",
         image_size, kl.symbol, kl.grid, kl.block, kl.cluster, kl.dynamic_smem, acc, c2[(size_t)7 * p.n + 519]);
  return 0;
}
