"""``python -m ayaka_b200``."""

from ayaka_b200.cli import main

raise SystemExit(main())
