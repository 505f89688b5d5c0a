/* A plain C consumer of the library: includes both headers, links against the shared
 * object and calls entry points that need no GPU.  Built and run by tests/test_abi.py. */
#include <stdio.h>
#include <string.h>

#include "paged_attn_b200.h"
#include "paged_attn_b200_host.h"

int main(void) {
  PaHostConfig cfg;
  pa_host_config_default(&cfg);
  if (pa_host_config_validate(&cfg) != PA_OK) return 1;
  const uint32_t toks[4] = {1u, 2u, 3u, 4u};
  const uint64_t h0 = pa_hash_tokens(toks, 4, 0), h1 = pa_hash_tokens(toks, 4, h0);
  int32_t ka, kb, qa, qb;
  if (pa_shard_head_ranges(1, 2, 32, 8, &ka, &kb, &qa, &qb) != PA_OK) return 2;
  if (pa_shard_head_ranges(0, 3, 32, 8, &ka, &kb, &qa, &qb) == PA_OK) return 3;
  if (strlen(pa_last_error_string()) == 0) return 4; /* the refusal left a message */
  pa_shard_head_ranges(1, 2, 32, 8, &ka, &kb, &qa, &qb);
  /* a null config is refused, not dereferenced */
  PagedAttnCache *cache = (PagedAttnCache *)0;
  if (pa_cache_create((const PagedAttnConfig *)0, 0, &cache) == PA_OK || cache) return 5;
  printf("version %d blocks %u block_size %u hash %d shard %d %d %d %d\n", (int)pa_version(),
         (unsigned)pa_host_config_num_blocks(&cfg), (unsigned)cfg.block_size, (int)(h0 != h1), (int)ka,
         (int)kb, (int)qa, (int)qb);
  return 0;
}
