/** Aggregate of the basic public definitions (types, logging, check macros). */
#pragma once
#include "megray/check.h"
#include "megray/config.h"
#include "megray/debug.h"
#include "megray/types.h"
