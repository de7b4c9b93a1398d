// Toy header of the packaging fixture: never compiled, only embedded.
#pragma once
#define TOY_SCALE_FACTOR 2.0f
