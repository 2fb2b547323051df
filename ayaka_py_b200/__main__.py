import sys

from .commands.cli import main

sys.exit(main())
