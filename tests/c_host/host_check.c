/* A C host of libb200base.so, as a maintainer of the reference would write one over the two headers: it must compile
 * as plain C99 with both headers, link against the library, and use the upper face (Artifact / Base) without a GPU.
 * What it checks follows the reference's own runtime tests: an artifact round trip through JSON, a Base whose memory is
 * initial_memory zero-extended (base/src/lib.rs:36-52), `execute` on an empty program succeeding, an out-of-range
 * function index reported as an Execution error (base/tests/integration.rs:2459-2469), and the native plugins' stage
 * tables.  Every declared entry point is referenced once so that a missing export fails at link time. */
#include <stdio.h>
#include <string.h>

#include "b200abi.h"
#include "b200base.h"

#define CHECK(cond)                                                         \
  do {                                                                      \
    if (!(cond)) {                                                          \
      fprintf(stderr, "host_check: line %d: %s\n", __LINE__, #cond);        \
      return 1;                                                             \
    }                                                                       \
  } while (0)

/* addresses of the lower-face entry points a host binds (never called here: they need a GPU) */
static const void *lower_face[] = {
    (const void *)cl_cuda_init,          (const void *)cl_cuda_cleanup,        (const void *)cl_cuda_create_buffer,
    (const void *)cl_cuda_free_buffer,   (const void *)cl_cuda_upload_ptr,     (const void *)cl_cuda_download_ptr,
    (const void *)cl_cuda_launch,        (const void *)cl_cuda_sync,           (const void *)cl_cuda_graph_launch,
    (const void *)cl_b200_launch,        (const void *)cl_b200_builtin_module, (const void *)cl_b200_stream_handle,
    (const void *)cl_b200_ipc_export,    (const void *)cl_b200_ipc_open,       (const void *)cl_b200_ipc_close,
    (const void *)cl_b200_comm_init,     (const void *)cl_b200_comm_all_gather, (const void *)cl_b200_argmax_noalloc,
};

int main(void) {
  const char *json =
      "{\"setup\":{\"cranelift_ir\":\"\",\"memory_size\":256,\"io_offsets\":{\"data_ptr\":24,\"data_len\":32,"
      "\"out_ptr\":40,\"out_len\":48},\"initial_memory\":[1,2,3,4]},\"main\":{\"fn_idx\":0,\"output\":[]},"
      "\"extras\":{\"prep\":{\"fn_idx\":1,\"output\":[]}}}";
  size_t i;
  for (i = 0; i < sizeof(lower_face) / sizeof(lower_face[0]); ++i) CHECK(lower_face[i] != NULL);

  B200Artifact *a = b200_artifact_from_json(json, (uint64_t)strlen(json));
  CHECK(a != NULL);
  CHECK(strcmp(b200_artifact_cranelift_ir(a), "") == 0);
  CHECK(b200_artifact_memory_size(a) == 256);
  uint64_t io[4];
  b200_artifact_io_offsets(a, io);
  CHECK(io[0] == 24 && io[1] == 32 && io[2] == 40 && io[3] == 48);
  uint64_t init_len = 0;
  const uint8_t *init = b200_artifact_initial_memory(a, &init_len);
  CHECK(init_len == 4 && init[0] == 1 && init[3] == 4);
  CHECK(b200_artifact_main_fn(a) == 0 && b200_artifact_extras_count(a) == 1);
  CHECK(strcmp(b200_artifact_extra_name(a, 0), "prep") == 0 && b200_artifact_extra_fn(a, 0) == 1);
  CHECK(b200_artifact_from_json("{", 1) == NULL);

  int32_t kind = -1;
  B200Base *b = b200_base_new(b200_artifact_cranelift_ir(a), b200_artifact_memory_size(a), io, init, init_len, &kind);
  CHECK(b != NULL);
  uint64_t mem_len = 0;
  uint8_t *mem = b200_base_memory(b, &mem_len);
  CHECK(mem_len >= 256 && mem[0] == 1 && mem[3] == 4 && mem[4] == 0 && mem[255] == 0);
  CHECK(b200_base_fn_count(b) == 0);
  /* an empty program has no functions: execute still succeeds, and still writes the four io words */
  uint8_t data[3] = {9, 8, 7}, out[5] = {0};
  CHECK(b200_base_execute_into(b, 0, data, sizeof data, out, sizeof out) == B200_OK);
  uint64_t word;
  memcpy(&word, mem + 32, 8);
  CHECK(word == sizeof data);
  memcpy(&word, mem + 48, 8);
  CHECK(word == sizeof out);
  b200_base_free(b);

  /* a native stage program: its stage table is the function table; an index past it is an Execution error */
  CHECK(b200_plugin_count() >= 3);
  uint32_t n = b200_plugin_fn_count("gptoss");
  CHECK(n >= 10 && strcmp(b200_plugin_fn_name("gptoss", 1), "load") == 0);
  b = b200_base_new("native:gptoss", 4096, io, NULL, 0, &kind);
  CHECK(b != NULL && b200_base_fn_count(b) == n);
  CHECK(b200_base_execute_into(b, n + 5, NULL, 0, NULL, 0) == B200_ERR_EXECUTION);
  CHECK(strlen(b200_last_error()) > 0 && cl_b200_last_error() != NULL);
  b200_base_free(b);
  CHECK(b200_base_new("native:no-such-plugin", 4096, io, NULL, 0, &kind) == NULL && kind == B200_ERR_CLIF_PARSE);
  b200_artifact_free(a);
  printf("host_check ok: %u plugins, gptoss has %u stages\n", b200_plugin_count(), n);
  return 0;
}
