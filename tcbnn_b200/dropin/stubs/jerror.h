// Stand-in for libjpeg error header (data.h:28); nothing is needed from it.
