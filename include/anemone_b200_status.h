/*
 * anemone_b200_status.h: how every host function of this library reports failure.
 *
 * Replaces the reference's include/anemone/status.h:23-38 (same enumerators, same values, so a caller
 * compiled against either header links against this library unchanged).
 *
 * Rules kept from that interface: a fallible function returns a result_status and delivers results only
 * through output parameters; on any failure its scalar outputs and launch tables are left untouched; bad
 * input is a status, never an exit() or abort().
 */
#ifndef ANEMONE_B200_STATUS_H
#define ANEMONE_B200_STATUS_H

#ifdef __cplusplus
extern "C" {
#endif

#ifndef MUST_CHECK
#define MUST_CHECK __attribute__((warn_unused_result))
#endif

typedef enum result_status {
	STATUS_OK = 0,
	STATUS_INVALID_ARGUMENT = 1,
	STATUS_OUT_OF_MEMORY = 2,
	STATUS_INPUT_OUTPUT_ERROR = 3,
	STATUS_CORRUPT_PACK = 4,
	STATUS_DEVICE_ERROR = 5,
	STATUS_TIMED_OUT = 6,
	STATUS_UNSUPPORTED = 7,
	STATUS_BUSY_VALUE = 8,
	STATUS_INJECTED_FAULT = 9,
	STATUS_COUNT = 10
} result_status;

/* Replaces status_text (include/anemone/status.h:38). Never NULL, also for values outside the enum. */
const char *status_text(result_status status);

#ifdef __cplusplus
}
#endif
#endif
