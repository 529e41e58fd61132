"""Entry point with the reference's contract: ``torchrun --nproc_per_node=N trainer.py --config X.json``."""
from lightron_b200.trainer import main

if __name__ == "__main__":
    main()
