"""B200-native epsilon self-join (FP16 in, FP32 accumulate): Python front end of libfasted.so."""
from ._lib import SelfJoin, JoinStats, FastedError, load, JOIN_DIST2, JOIN_NO_SORT, JOIN_KEEP_NORMS, JOIN_SYMMETRIC  # noqa: F401
from .find_pairs import load_findpairs, Results, mmaShape, RerunnablePairsFinder, compute_selectivity  # noqa: F401
