// Empty stand-in for the reference's src/common/rand.cuh (cuRAND device state): the first-level hash functions do not
// use it.  Found before the real file because this folder precedes the reference's src/ on the include path.
#pragma once
