// Source compatibility: the reference ships collectives as <rocshmem/rocshmem_COLL.hpp>
// (include/rocshmem/rocshmem_COLL.hpp). Programs written against it include this file unchanged.
// The whole typed surface is generated from the type tables of rocshmem.h, so every one of the
// reference's per-family headers forwards to it.
#pragma once
#include "rocshmem.h"
