/*
 * ref_stubs.c: empty stand-ins for functions the reference's storage files name but the map reader never calls (its
 * direct-read storage pulls in the native pack and the n-gram tables). TEST INFRASTRUCTURE: linked only into
 * oracle/_ref/libanemone_ref.so so that it loads; none of them is ever called, none holds reference code.
 */
void engram_close(void) {}
void engram_description_of(void) {}
void engram_hashing_equal(void) {}
void engram_open(void) {}
void pack_close(void) {}
void pack_extents_of(void) {}
void pack_header_of(void) {}
void pack_open_entry(void) {}
void pack_units_of(void) {}
