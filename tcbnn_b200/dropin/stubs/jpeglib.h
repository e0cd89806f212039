// Stand-in for libjpeg, which the reference data.h includes (data.h:27) but this build never calls:
// images are synthetic.
