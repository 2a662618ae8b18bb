"""Native (C++) host runtime: indexed-dataset reader / batch prefetcher and helpers."""
