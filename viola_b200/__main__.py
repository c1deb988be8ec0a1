from .parallel.launch import main

main()
