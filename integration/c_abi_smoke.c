/* Plain C99 translation unit: proves that include/xnor_b200.h is a C header (no C++-isms) and that the host-only entry
 * points link and run without a GPU.  Built and run by tests/test_boundary_compile.py. */
#include <stdio.h>
#include <string.h>

#include "xnor_b200.h"

int main(void)
{
	xnor_b200_conv_desc d;
	xnor_b200_conv_geom g;
	memset(&d, 0, sizeof d);
	d.batch = 1; d.c = 256; d.h = 26; d.w = 26; d.n = 512; d.size = 3; d.stride = 1; d.pad = 1; d.activation = XNOR_B200_LEAKY;
	if (xnor_b200_conv_geometry(&d, &g) != XNOR_B200_OK) { return 1; }
	/* the always-add alignment of make_convolutional_layer / binary_align_weights: K = 2304 -> 2560, N = 676 -> 704 */
	if (g.k != 2304 || g.new_lda != 2560 || g.bit_align != 704 || g.n_out != 676) { return 2; }
	if (xnor_b200_scratch_bytes(&d) < g.packed_input_bytes) { return 3; }
	d.stride = 0;
	if (xnor_b200_conv_geometry(&d, &g) != XNOR_B200_ERR_INVALID) { return 4; }
	printf("%s|%s\n", xnor_b200_strerror(XNOR_B200_OK), xnor_b200_strerror(XNOR_B200_ERR_SCRATCH));
	return 0;
}
