// Source compatibility: the reference ships signalling operations as <rocshmem/rocshmem_SIG_OP.hpp>
// (include/rocshmem/rocshmem_SIG_OP.hpp). Programs written against it include this file unchanged.
// The whole typed surface is generated from the type tables of rocshmem.h, so every one of the
// reference's per-family headers forwards to it.
#pragma once
#include "rocshmem.h"
