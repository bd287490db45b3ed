"""Stand-in for ``imageio`` (image file reader of the reference datasets; unused with synthetic batches)."""
