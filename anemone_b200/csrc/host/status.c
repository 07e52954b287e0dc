/* status.c: the one English phrase per status (replaces the reference's source/status.c). */
#include "anemone_b200_status.h"

const char *status_text(result_status status)
{
	static const char *const texts[STATUS_COUNT] = {
		"ok",	       "invalid argument", "out of memory", "input/output error", "corrupt pack",
		"device error", "timed out",	   "unsupported",   "busy",		  "injected fault"
	};
	return (unsigned)status < STATUS_COUNT ? texts[status] : "unknown status";
}
