"""``python -m forge_engine_b200`` is the ``forge-engine`` command."""

from .cli import main

raise SystemExit(main())
