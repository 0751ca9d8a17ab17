/* The structural matchers from plain C, with no GPU: a node list written to a file as
 *   int32 n_nodes, n_in, n_shape, n_arg; int32 op[n]; int32 in_off[n+1]; int32 in_node[n_in];
 *   int32 shape_off[n+1]; int64 shape[n_shape]; int32 arg_off[n+1]; double arg[n_arg]
 * is read back into lmb200_node_list and handed to the matcher named on the command line.
 * usage: cabi_match <file> <decoder|step|encoder> <output_id>      prints one JSON line, exit 0; no match: exit 3 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "luminal_b200.h"

static void* read_block(FILE* f, size_t bytes) {
  void* p = malloc(bytes ? bytes : 1);
  if (!p || (bytes && fread(p, 1, bytes, f) != bytes)) {
    fprintf(stderr, "short file\n");
    exit(65);
  }
  return p;
}

int main(int argc, char** argv) {
  FILE* f;
  int32_t head[4], n, output_id, rc, k;
  lmb200_node_list list;
  lmb200_model_config cfg;
  lmb200_decoder_match info;
  lmb200_encoder_match einfo;
  int32_t* nodes;
  char* names;
  if (argc != 4) return 64;
  f = fopen(argv[1], "rb");
  if (!f || fread(head, sizeof(int32_t), 4, f) != 4) return 65;
  n = head[0];
  memset(&list, 0, sizeof list);
  list.n_nodes = n;
  list.op = (const int32_t*)read_block(f, sizeof(int32_t) * (size_t)n);
  list.in_off = (const int32_t*)read_block(f, sizeof(int32_t) * (size_t)(n + 1));
  list.in_node = (const int32_t*)read_block(f, sizeof(int32_t) * (size_t)head[1]);
  list.shape_off = (const int32_t*)read_block(f, sizeof(int32_t) * (size_t)(n + 1));
  list.shape = (const int64_t*)read_block(f, sizeof(int64_t) * (size_t)head[2]);
  list.arg_off = (const int32_t*)read_block(f, sizeof(int32_t) * (size_t)(n + 1));
  list.arg = (const double*)read_block(f, sizeof(double) * (size_t)head[3]);
  fclose(f);
  output_id = (int32_t)atoi(argv[3]);
  nodes = (int32_t*)calloc((size_t)n, sizeof(int32_t));
  names = (char*)calloc((size_t)n * 64 + 256, 1);
  memset(&cfg, 0, sizeof cfg);
  memset(&info, 0, sizeof info);
  memset(&einfo, 0, sizeof einfo);
  if (strcmp(argv[2], "decoder") == 0)
    rc = lmb200_match_decoder(&list, output_id, &cfg, &info, nodes, n, names, (int64_t)n * 64 + 256);
  else if (strcmp(argv[2], "step") == 0)
    rc = lmb200_match_whisper_step(&list, output_id, &cfg, &info, nodes, n, names, (int64_t)n * 64 + 256, NULL, 0);
  else
    rc = lmb200_match_whisper_encoder(&list, output_id, &einfo, nodes, n, names, (int64_t)n * 64 + 256);
  if (rc != LMB200_OK) {
    fprintf(stderr, "%d: %s\n", (int)rc, lmb200_last_error());
    return rc == LMB200_ENOMATCH ? 3 : 2;
  }
  if (strcmp(argv[2], "encoder") == 0) {
    printf("{\"d_model\": %d, \"heads\": %d, \"layers\": %d, \"ffn\": %d, \"n_mels\": %d, \"batch\": %d, \"frames\": %d, \"mel\": %d, "
           "\"n_weights\": %d, \"nodes\": [",
           (int)einfo.d_model, (int)einfo.heads, (int)einfo.layers, (int)einfo.ffn, (int)einfo.n_mels, (int)einfo.batch,
           (int)einfo.frames, (int)einfo.mel_node, (int)einfo.n_weights);
    for (k = 0; k < einfo.n_weights; ++k) printf("%s%d", k ? ", " : "", (int)nodes[k]);
  } else {
    printf("{\"arch\": %d, \"n_layers\": %d, \"hidden\": %d, \"n_heads\": %d, \"n_kv_heads\": %d, \"intermediate\": %d, \"vocab\": %d, "
           "\"batch\": %d, \"seq\": %d, \"prev_seq\": %d, \"tokens\": %d, \"n_weights\": %d, \"nodes\": [",
           (int)info.arch, (int)cfg.n_layers, (int)cfg.hidden, (int)cfg.n_heads, (int)cfg.n_kv_heads, (int)cfg.intermediate,
           (int)cfg.vocab, (int)info.batch, (int)info.seq, (int)info.prev_seq, (int)info.tokens_node, (int)info.n_weights);
    for (k = 0; k < info.n_weights; ++k) printf("%s%d", k ? ", " : "", (int)nodes[k]);
  }
  printf("], \"first_name\": \"%.*s\"}\n", (int)strcspn(names, "\n"), names);
  return 0;
}
