// Force-included (-include) when the reference's sources are compiled on Linux: the only MSVC
// library call its dense core makes that glibc does not have.  The reference's files stay as
// they are.
#pragma once
#include <cstdio>
#define _fseeki64 fseeko64
#define _ftelli64 ftello64
