"""``python -m atom_b200.weights --config DIR_OR_JSON --seed N --out DIR`` writes a model folder
with seeded random weights (see random_init.main)."""
from .random_init import main

raise SystemExit(main())
