/* placeholder translation unit: the GGA oracle is added with the GGA kernels */
int sqo_gga_placeholder(void) { return 0; }
