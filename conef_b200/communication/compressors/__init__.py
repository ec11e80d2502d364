"""Reference import names for the error compressors."""
