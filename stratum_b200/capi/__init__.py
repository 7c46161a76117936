"""The C interface: stratum.h and stratum_capi.c (a layer that forwards to `host` inside an interpreter), and
`build.library()` that compiles them."""
