"""`python inference.py --checkpoint <exp_dir> --prompt "..."` — see adana_b200/inference.py."""
from adana_b200.inference import main

if __name__ == "__main__":
    raise SystemExit(main())
