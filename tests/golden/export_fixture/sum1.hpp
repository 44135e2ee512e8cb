// N2D2 auto-generated file.

#ifndef N2D2_EXPORTC_SUM1_LAYER_H
#define N2D2_EXPORTC_SUM1_LAYER_H

#include "../../include/typedefs.h"
#include "../../include/utils.h"
#define SUM1_NB_INPUTS 2
#define SUM1_NB_OUTPUTS 16
#define SUM1_NB_CHANNELS 32
#define SUM1_OUTPUTS_WIDTH 4
#define SUM1_OUTPUTS_HEIGHT 4
#define SUM1_CHANNELS_WIDTH 4
#define SUM1_CHANNELS_HEIGHT 4

#define SUM1_ACTIVATION Rectifier
static const N2D2_Export::SingleShiftScaling<1> SUM1_SCALING;

#define SUM1_ELEM_OP Sum
#define SUM1_ELEM_COEFF_MODE PerLayer

#endif // N2D2_EXPORTC_SUM1_LAYER_H
