import sys

from .evidence import main

sys.exit(main())
