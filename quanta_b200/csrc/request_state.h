// The per-request state slot: one fixed-size record on the device for every live request.
//
// The reference keeps this per stream on the host (src/quanta/shim/omlx.py:1055-1081 `_StreamState`:
// sampling options, rng key, generated ids; src/quanta/paged/paged_kv_cache.py:82-91 `SeqHandle`:
// length).  Here the part of it that a step needs lives on the device, so that a decode step and its
// sampling read nothing from the host but the block tables: the record is written once when a
// request takes the slot (one small copy), the step advances the position, the sampler reads its
// options from it, counts the draw and leaves the sampled token in it, and the next step may take
// its token from there before the host has seen it.  A freed slot is all zeros.
#pragma once

#define QB_SLOT_WORDS 16          // int32 words a record; floats are stored as their bit patterns
#define QB_SLOT_LIVE 0            // 1 while a request holds the slot
#define QB_SLOT_POSITION 1        // tokens of the request in the cache
#define QB_SLOT_PROMPT 2          // length of its prompt
#define QB_SLOT_DRAWN 3           // tokens sampled so far = number of the next draw
#define QB_SLOT_LAST 4            // the token sampled last
#define QB_SLOT_SEED_LO 5
#define QB_SLOT_SEED_HI 6
#define QB_SLOT_TOP_K 7           // 0: off
#define QB_SLOT_TEMPERATURE 8     // float; <= 0: greedy
#define QB_SLOT_TOP_P 9           // float; outside (0, 1): off
#define QB_SLOT_MIN_P 10          // float; 0: off
