"""B200-native compressed linear algebra for SystemDS column groups (matrix-multiply path)."""
from .cmb import (CHAIN_XtXv, CHAIN_XtwXv, CLALibDecompress, CLALibLeftMultBy, CLALibMatrixMult, CLALibMMChain,
                  CLALibRightMultBy,
                  CLALibTSMM, CompressedMatrixBlock)
from .native import CLAError

__all__ = ["CompressedMatrixBlock", "CLALibRightMultBy", "CLALibLeftMultBy", "CLALibTSMM", "CLALibMMChain",
           "CLALibDecompress", "CLALibMatrixMult", "CLAError", "CHAIN_XtXv", "CHAIN_XtwXv"]
