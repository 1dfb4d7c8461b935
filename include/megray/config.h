/**
 * Build configuration.  The reference generates this file from config.h.in
 * (reference include/megray/config.h.in:15-22); here the switches are plain
 * compiler definitions (-DMEGRAY_WITH_CUDA ...) with the defaults below.
 */
#pragma once

#ifndef MEGRAY_LOG_LEVEL
#define MEGRAY_LOG_LEVEL 2 /* compile-time floor: WARN; MEGRAY_LOG_LEVEL env can raise it */
#endif

/* MEGRAY_WITH_CUDA, MEGRAY_WITH_NCCL, MEGRAY_WITH_NVL, MEGRAY_WITH_SHM are set by the build.
 * MEGRAY_WITH_UCX, MEGRAY_WITH_RCCL, MEGRAY_WITH_HIP are never set on this platform. */
