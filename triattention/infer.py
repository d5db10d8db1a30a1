"""``python -m triattention.infer`` — the reference's entry point (infer.py:8-18), same flags, on the sm_100a kernels."""
from triattention_b200.infer import main

if __name__ == "__main__":
    main()
