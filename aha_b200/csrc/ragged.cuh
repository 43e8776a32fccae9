// ragged.cuh -- the description of one engine step as the kernels of the ragged (varlen) path see it: the tokens of all
// entries packed back to back -- a portion of a prompt beside single decoded tokens -- each entry with its sequence slot, the
// position of its first token and its page table.  Every kernel of that path takes this struct; none assumes equal lengths.
#pragma once
#include "attention.cuh"   // kPage / kPageShift: the KV page size of the library

namespace aha {

struct RaggedBatch {
    int T = 0;                        // packed tokens of the step
    int E = 0;                        // entries (sequences taking part)
    const uint32_t* tokens = nullptr; // [T] token ids
    const int* tok_entry = nullptr;   // [T] entry of a packed token
    const int* tok_pos = nullptr;     // [T] position of the token in its sequence (counts from 0)
    const int* ent_start = nullptr;   // [E + 1] packed offset of an entry's first token
    const int* ent_pos0 = nullptr;    // [E] tokens the sequence held before this step
    const int* ent_slot = nullptr;    // [E] state slot of the sequence
    const int* page_tables = nullptr; // [slots][max_pages] logical page -> physical page
    int max_pages = 0;
};

}  // namespace aha
