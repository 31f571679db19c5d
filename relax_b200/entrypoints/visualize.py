"""Launch the rollout result viewer (relax/entrypoints/visualize.py): ``python -m relax_b200.entrypoints.visualize --dir dumps/``."""
from ..utils.visualize import main

if __name__ == "__main__":
    raise SystemExit(main())
