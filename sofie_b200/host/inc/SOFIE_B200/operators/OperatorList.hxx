// Every operator of the B200 target.
#pragma once
#include "SOFIE_B200/operators/ROperator_Conv.hxx"
#include "SOFIE_B200/operators/ROperator_Elementwise.hxx"
#include "SOFIE_B200/operators/ROperator_Gemm.hxx"
#include "SOFIE_B200/operators/ROperator_Quantized.hxx"
#include "SOFIE_B200/operators/ROperator_Sequence.hxx"
