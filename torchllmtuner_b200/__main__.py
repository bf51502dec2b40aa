from .trainer.cli import main

raise SystemExit(main())
