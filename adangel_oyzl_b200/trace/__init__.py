"""Prepared-sample persistence and preparation (the callers in front of the GEMM hot path)."""

from ..schema import PreparedInputs, validate_prepared
from .storage import (MANIFEST_VERSION, PREPARED_FORMAT, load_prepared, save_prepared, sha256_file,
                      validate_manifest, write_manifest)

__all__ = ["PreparedInputs", "validate_prepared", "MANIFEST_VERSION", "PREPARED_FORMAT", "load_prepared",
           "save_prepared", "sha256_file", "validate_manifest", "write_manifest"]
