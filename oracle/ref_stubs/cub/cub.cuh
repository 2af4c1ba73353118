// Empty stand-in: the hash functions compiled for the host use nothing from CUB.
#pragma once
