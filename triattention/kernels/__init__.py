"""Host executors and the extension loader under the reference's module paths."""
