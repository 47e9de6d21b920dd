// What this build of the library is and what it contains, as preprocessor constants (reference:
// cmake/rocshmem_config.h.in, a list of the CMake options the library was configured with). Almost every choice
// that is a build option there is made at run time here, so the constants below describe the one build there is.
#pragma once

#define ROCSHMEM_B200_VERSION_MAJOR 0
#define ROCSHMEM_B200_VERSION_MINOR 1
#define ROCSHMEM_B200_VERSION_PATCH 0
#define ROCSHMEM_B200_VERSION_STRING "0.1.0"

// Always present.
#define ROCSHMEM_HAS_PEER_MAPPING 1        // NVLink peer loads / stores on one virtual window (the reference's USE_IPC)
#define ROCSHMEM_HAS_REVERSE_OFFLOAD 1     // host proxy thread; switched on with ROCSHMEM_USE_PROXY (USE_RO)
#define ROCSHMEM_HAS_MESSAGE_COALESCING 1  // ROCSHMEM_USE_WF_COAL (USE_WF_COAL)
#define ROCSHMEM_HAS_THREAD_MULTIPLE 1     // host API callable from several threads (USE_THREADS)
#define ROCSHMEM_HAS_SHAREABLE_CONTEXTS 1  // (USE_SHARED_CTX)
#define ROCSHMEM_HAS_NVLS 1                // multimem reductions and broadcast where the driver offers multicast
#define ROCSHMEM_SINGLE_NODE 1             // one NVSwitch domain, no NIC path (USE_SINGLE_NODE)
// Never present: a NIC backend (USE_GPU_IB, USE_DC) and the AMD-specific heap kinds and cache flushes.
#define ROCSHMEM_HAS_NIC_BACKEND 0

// Per translation unit, chosen by the program that includes the device API:
//   -DROCSHMEM_PROFILE      count device-side API calls and time the reverse-offload path (PROFILE)
//   -DROCSHMEM_DEBUG_PRINT  device printf tracing through ROCSHMEM_GPU_DPRINTF (DEBUG)

// The reference's bare option names, for programs that test them with #ifdef. Opt-in because they are short names
// in the global macro namespace.
#ifdef ROCSHMEM_REFERENCE_CONFIG_NAMES
#define USE_IPC
#define USE_RO
#define USE_WF_COAL
#define USE_THREADS
#define USE_SHARED_CTX
#define USE_SINGLE_NODE
#ifdef ROCSHMEM_PROFILE
#define PROFILE
#endif
#ifdef ROCSHMEM_DEBUG_PRINT
#define DEBUG
#endif
#endif
