/* Drop-in name: programs written against the ASPEN reference include "aspen.h" and nothing else.
 * The API itself is declared in aspen_b200.h.  This forwarder also supplies what the reference's
 * public header gives its users in passing and their sources rely on (ref: include/aspen.h:3-48):
 * the C library headers it pulls in (main.c uses FILE, struct timeval, gettimeofday, strcmp, atoi
 * without including anything itself) and the coloured print macros. */
#ifndef ASPEN_H_FORWARD_
#define ASPEN_H_FORWARD_

#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif
#include <assert.h>
#include <ctype.h>
#include <float.h>
#include <limits.h>
#include <math.h>
#include <pthread.h>
#include <sched.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>
#include <time.h>
#include <unistd.h>

#include "aspen_b200.h"

/* ref: include/aspen.h:34-48.  SUPPRESS_OUTPUT != 0 silences everything but a one-line error note. */
#define ASPEN_COLOURED_(stream, code, ...) \
    do { fprintf(stream, "\033[0;" code "m"); fprintf(stream, __VA_ARGS__); fprintf(stream, "\033[0m"); } while (0)
#if !defined(SUPPRESS_OUTPUT) || SUPPRESS_OUTPUT == 0
#define PRTF(...) printf(__VA_ARGS__)
#define ERROR_PRTF(...) \
    do { fprintf(stderr, "\033[0;31m(%s:%d)", __FILE__, __LINE__); fprintf(stderr, __VA_ARGS__); fprintf(stderr, "\033[0m"); } while (0)
#define RED_PRTF(...) ASPEN_COLOURED_(stdout, "31", __VA_ARGS__)
#define GREEN_PRTF(...) ASPEN_COLOURED_(stdout, "32", __VA_ARGS__)
#define YELLOW_PRTF(...) ASPEN_COLOURED_(stdout, "33", __VA_ARGS__)
#define BLUE_PRTF(...) ASPEN_COLOURED_(stdout, "34", __VA_ARGS__)
#else
#define PRTF(...) do { } while (0)
#define ERROR_PRTF(...) do { fprintf(stderr, "\033[0;31mASPEN: An error has occured.\033[0m"); } while (0)
#define RED_PRTF(...) do { } while (0)
#define GREEN_PRTF(...) do { } while (0)
#define YELLOW_PRTF(...) do { } while (0)
#define BLUE_PRTF(...) do { } while (0)
#endif

#endif
