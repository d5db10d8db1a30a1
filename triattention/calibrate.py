"""``python -m triattention.calibrate`` — the reference's entry point (calibrate.py:32-73), same flags and output format,
with the whole grid evaluated in one pass per layer."""
from triattention_b200.calibrate import W4, W8, Calibration, grid, head_errors, load_samples, main  # noqa: F401

if __name__ == "__main__":
    main()
