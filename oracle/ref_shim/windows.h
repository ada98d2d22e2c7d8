// TEST INFRASTRUCTURE ONLY: the one type a reference header (its memory-mapped file class, not used
// here) names from this platform header.
#pragma once
typedef void* HANDLE;
