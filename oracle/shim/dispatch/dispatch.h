/* Empty stand-in for Apple's libdispatch header: the reference's functions below
 * main() do not use it; the driver parallelises over population pairs itself. */
#ifndef EGG_SHIM_DISPATCH_H
#define EGG_SHIM_DISPATCH_H
#endif
