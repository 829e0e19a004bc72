// Prints, as JSON, the size of the reference engine's weight / activation
// structs and the byte offsets of the fields its MoE entry point reads and
// writes.  Compiled against the reference's own header (REF_TYPES_HEADER), so
// that nothing of that header has to live in this repository.  Test tooling.
#include <cstddef>
#include <cstdio>

#include REF_TYPES_HEADER

int main() {
  printf("{\n");
  printf("  \"sizeof_GpuWeights\": %zu,\n", sizeof(GpuWeights));
  printf("  \"sizeof_GpuActivations\": %zu,\n", sizeof(GpuActivations));
#define W(f) printf("  \"w." #f "\": %zu,\n", offsetof(GpuWeights, f))
#define A(f) printf("  \"a." #f "\": %zu,\n", offsetof(GpuActivations, f))
  W(enable_moe);
  W(expert_count);
  W(d_router_weights);
  W(d_expert_gate);
  W(d_expert_up);
  W(d_expert_down);
  A(d_ffn_output);
  A(d_residual_out);
  A(d_router_logits);
  A(d_expert_first);
  A(d_expert_second);
  A(d_weight_first);
  A(d_weight_second);
  A(d_expert_histogram);
  printf("  \"ok\": 1\n}\n");
  return 0;
}
