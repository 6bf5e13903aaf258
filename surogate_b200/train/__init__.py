"""Training workflows (SFT / pre-training), schedules, monitors, logging.  Parity: surogate/train/."""
