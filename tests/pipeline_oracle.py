"""The record-level oracle lives with the other oracle modules; kept here for the tests that import it by this name."""
from oracle.pipeline import PipelineOracle  # noqa: F401
